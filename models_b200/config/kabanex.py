"""Typed configuration of the Kabanex decoder, read from the keys of its own config.json.

A Kabanex layer has ONE layer norm whose rows feed a mixer and (optionally) a dense feed-forward
side by side: x += mixer(norm(x)) + feed_forward(norm(x)).  Its mixer "parallel" is itself two
mixers side by side: a grouped-query attention with a sliding window that also keeps the first
positions of the sequence, partial rotary positions, softmax weights mixed across heads, and a
per-head output gate; and a minGRU recurrence.  Their results are added with one scale each.

config.json (every size and constant of a model is here or is a tensor's shape):

    {"architecture": "Kabanex", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s,
                                    "rot": {"dims": r, "base": b}, "mask": {"size": n, "keep_first": f}},
                           "right": {"width": R}, "left_scale": a, "right_scale": c},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Tensors: `embed`, `head`, `final.norm` (+ `.b`), and per layer i under `l<i>.`: `norm1` (+ `.b`),
`mix.left.{q,k,v,talk,g,o}`, `mix.right.{z,x,g,o}` with biases `mix.right.{z,x}.b`, `mlp.{up,down}`.
Linear weights are [out, in].
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError
from .specs import (
    DenseFeedForwardSpec,
    EmbeddingSpec,
    HeadSpec,
    LayerNormSpec,
    MinGruSpec,
    ModelSpec,
    ParallelBlockSpec,
    RopeSpec,
    ScheduleEntry,
    SideBySideSpec,
    TalkingAttentionSpec,
)

ARCHITECTURE = "Kabanex"
# The configuration states no longest sequence: positions are limited by the cache an engine is made with.
UNLIMITED_POSITIONS = 1 << 30


def _get(raw: Mapping[str, Any], key: str, where: str):
    if not isinstance(raw, Mapping) or raw.get(key) is None:
        raise ConfigError(f"config.json: {where} needs the key {key!r}")
    return raw[key]


def _int(raw, key: str, where: str, least: int = 1) -> int:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {least}, got {value!r}")
    return value


def _float(raw, key: str, where: str, positive: bool = False) -> float:
    value = _get(raw, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a finite number{' > 0' if positive else ''}, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class KabanexAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int  # 0: no rotation
    rot_base: float
    window: Optional[int]
    keep_first: int


@dataclass(frozen=True)
class KabanexLayer:
    attention: KabanexAttention
    recurrent_width: int
    left_scale: float
    right_scale: float
    ff: Optional[int]  # None: no feed-forward in this layer


@dataclass(frozen=True)
class KabanexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[KabanexLayer, ...]

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "KabanexConfig":
        vocab = _int(raw, "vocab", "the model")
        width = _int(raw, "width", "the model")
        eps = _float(_get(raw, "norm", "the model"), "eps", "norm", positive=True)
        listed = _get(raw, "layers", "the model")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            if kind != "parallel":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: parallel)")
            mixer = _get(entry, "mixer", where)
            left = _get(mixer, "left", where + ".mixer")
            lw = where + ".mixer.left"
            heads, kv_heads = _int(left, "heads", lw), _int(left, "kv_heads", lw)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {lw}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
            dim, vdim = _int(left, "dim", lw), _int(left, "vdim", lw)
            rot = left.get("rot")
            rot_dims, rot_base = 0, 1.0
            if rot is not None:
                rot_dims = _int(rot, "dims", lw + ".rot", least=0)
                if rot_dims:
                    rot_base = _float(rot, "base", lw + ".rot", positive=True)
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"config.json: {lw}.rot.dims must be even and at most dim ({dim}), got {rot_dims}")
            mask = left.get("mask")
            window, keep_first = None, 0
            if mask is not None:
                window = _int(mask, "size", lw + ".mask")
                keep_first = _int(mask, "keep_first", lw + ".mask", least=0) if mask.get("keep_first") is not None else 0
            attention = KabanexAttention(heads, kv_heads, dim, vdim, _float(left, "scale", lw), rot_dims, rot_base, window,
                                         keep_first)
            right = _get(mixer, "right", where + ".mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                mlp_kind = _get(mlp, "kind", where + ".mlp")
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp_kind!r} is not built (known: dense)")
                ff = _int(mlp, "ff", where + ".mlp")
            layers.append(KabanexLayer(attention, _int(right, "width", where + ".mixer.right"),
                                       _float(mixer, "left_scale", where + ".mixer"),
                                       _float(mixer, "right_scale", where + ".mixer"), ff))
        return KabanexConfig(str(raw.get("architecture", ARCHITECTURE)), vocab, width, eps, tuple(layers))

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            a = layer.attention
            left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.rot_dims:
                left["rot"] = {"dims": a.rot_dims, "base": a.rot_base}
            if a.window is not None:
                left["mask"] = {"size": a.window, "keep_first": a.keep_first}
            layers.append({
                "type": "parallel",
                "mixer": {"left": left, "right": {"width": layer.recurrent_width}, "left_scale": layer.left_scale,
                          "right_scale": layer.right_scale},
                "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff},
            })
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": layers}

    def model_spec(self) -> ModelSpec:
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            a = layer.attention
            rope = RopeSpec(rotary_dim=a.rot_dims, theta=a.rot_base, pairing="half") if a.rot_dims else None
            left = TalkingAttentionSpec(
                hidden_size=self.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim,
                scale=a.scale, position=rope, window=a.window, keep_first=a.keep_first, gated=True,
                weights={"q": p + "mix.left.q", "k": p + "mix.left.k", "v": p + "mix.left.v", "talk": p + "mix.left.talk",
                         "gate": p + "mix.left.g", "o": p + "mix.left.o"})
            right = MinGruSpec(
                hidden_size=self.width, state_size=layer.recurrent_width,
                weights={"z": p + "mix.right.z", "z_bias": p + "mix.right.z.b", "x": p + "mix.right.x",
                         "x_bias": p + "mix.right.x.b", "gate": p + "mix.right.g", "o": p + "mix.right.o"})
            feed_forward = None
            if layer.ff is not None:
                feed_forward = DenseFeedForwardSpec(self.width, layer.ff, "relu2",
                                                    {"up": p + "mlp.up", "down": p + "mlp.down"})
            blocks.append(ParallelBlockSpec(
                mixer=SideBySideSpec(left, right, layer.left_scale, layer.right_scale),
                feed_forward=feed_forward,
                norm=LayerNormSpec(self.width, self.norm_eps, {"weight": p + "norm1", "bias": p + "norm1.b"})))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, self.width, 1.0, {"weight": "embed"}),
            layers=tuple(blocks),
            schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            final_norm=LayerNormSpec(self.width, self.norm_eps, {"weight": "final.norm", "bias": "final.norm.b"}),
            head=HeadSpec(self.vocab, self.width, False, {"weight": "head"}),
        )
