"""Typed configuration of the Lovurax decoder, read from the keys of its own config.json.

A Lovurax layer is pre-norm with gated residuals: h = rmsnorm(x); x += sigmoid(G h + b) * mixer(h); then the
same with a second norm and gate for a dense feed-forward, if the layer has one.  Every layer names its mixer:

  "retention"         linear attention with a fixed decay per head, rotary positions on part of a head, a
                      float32 state per sequence instead of a cache;
  "attention"         grouped-query attention without rotation or softmax: query/key norm, a query temperature
                      that grows with the position, a distance term per head, sigmoid weights, an output gate;
  "latent_attention"  softmax attention whose keys and values are expanded from one cached low-rank row.

The feed-forward is down(xielu(up(h))) with two learned shape numbers.  The output reuses the embedding
table, times `logit_scale`.

config.json (every size and constant of a model is here or is a tensor's shape):

    {"architecture": "Lovurax", "vocab": V, "width": W, "norm": {"eps": e}, "logit_scale": s,
     "layers": [{"type": "retention", "mixer": {"heads": H, "dim": D, "vdim": Dv, "decay": [d_0, ...],
                                                "rot": {"dims": r, "base": b}}, "mlp": {"kind": "dense", "ff": F} | null},
                {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": s,
                                                "q_temp": {"coef": c, "every": n}}, "mlp": ...},
                {"type": "latent_attention", "mixer": {"heads": H, "dim": D, "vdim": Dv, "kv_rank": R, "scale": s},
                 "mlp": ...}, ...]}

Tensors: `embed`, `final.norm`, and per layer i under `l<i>.`: `norm1`, `rg1`, `rg1.b`, with a feed-forward also
`norm2`, `rg2`, `rg2.b`, `mlp.{up,down,act}`; `mix.{q,k,v,g,o}` (retention), `mix.{q,k,v,q.norm,k.norm,pb,g,o}`
(attention), `mix.{q,dkv,dkv.norm,uk,uv,g,o}` (latent attention).  Linear weights are [out, in].
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .kabanex import UNLIMITED_POSITIONS, _float, _get, _int
from .llama import ConfigError
from .specs import (
    DenseFeedForwardSpec,
    EmbeddingSpec,
    GatedResidualBlockSpec,
    HeadSpec,
    LatentAttentionSpec,
    ModelSpec,
    NormSpec,
    RetentionSpec,
    RopeSpec,
    ScheduleEntry,
    SigmoidAttentionSpec,
)

ARCHITECTURE = "Lovurax"
# The distance term of the sigmoid attention: slope_h = 2^(-SLOPE_EXPONENT * (h + 1) / heads).
SLOPE_EXPONENT = 8.0
MIXERS = ("retention", "attention", "latent_attention")


@dataclass(frozen=True)
class LovuraxRetention:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_dims: int  # 0: no rotation
    rot_base: float


@dataclass(frozen=True)
class LovuraxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float  # 0: no query temperature
    temp_every: int


@dataclass(frozen=True)
class LovuraxLatentAttention:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float


@dataclass(frozen=True)
class LovuraxLayer:
    type: str
    mixer: object
    ff: Optional[int]  # None: no feed-forward in this layer


def _rotation(mixer, where: str, dim: int):
    rot = mixer.get("rot")
    if rot is None:
        return 0, 1.0
    dims = _int(rot, "dims", where + ".rot", least=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
    return dims, (_float(rot, "base", where + ".rot", positive=True) if dims else 1.0)


def _mixer(kind: str, mixer, where: str):
    heads, dim, vdim = _int(mixer, "heads", where), _int(mixer, "dim", where), _int(mixer, "vdim", where)
    if kind == "retention":
        decay = _get(mixer, "decay", where)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")
        values = []
        for n, d in enumerate(decay):
            if isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 <= d <= 1.0:
                raise ConfigError(f"config.json: {where}.decay[{n}] must be a number in [0, 1], got {d!r}")
            values.append(float(d))
        rot_dims, rot_base = _rotation(mixer, where, dim)
        return LovuraxRetention(heads, dim, vdim, tuple(values), rot_dims, rot_base)
    if kind == "attention":
        kv_heads = _int(mixer, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        temp = mixer.get("q_temp")
        coef, every = 0.0, 1
        if temp is not None:
            coef = _float(temp, "coef", where + ".q_temp")
            value = _get(temp, "every", where + ".q_temp")
            if isinstance(value, float) and value.is_integer():
                value = int(value)
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ConfigError(f"config.json: {where}.q_temp.every must be an integer >= 1, got {value!r}")
            every = value
        return LovuraxAttention(heads, kv_heads, dim, vdim, _float(mixer, "scale", where), coef, every)
    return LovuraxLatentAttention(heads, dim, vdim, _int(mixer, "kv_rank", where), _float(mixer, "scale", where))


@dataclass(frozen=True)
class LovuraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[LovuraxLayer, ...]

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "LovuraxConfig":
        vocab = _int(raw, "vocab", "the model")
        width = _int(raw, "width", "the model")
        eps = _float(_get(raw, "norm", "the model"), "eps", "norm", positive=True)
        logit_scale = _float(raw, "logit_scale", "the model") if raw.get("logit_scale") is not None else 1.0
        listed = _get(raw, "layers", "the model")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not built (known: {', '.join(MIXERS)})")
            mixer = _mixer(kind, _get(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                mlp_kind = _get(mlp, "kind", where + ".mlp")
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp_kind!r} is not built (known: dense)")
                ff = _int(mlp, "ff", where + ".mlp")
            layers.append(LovuraxLayer(kind, mixer, ff))
        return LovuraxConfig(str(raw.get("architecture", ARCHITECTURE)), vocab, width, eps, logit_scale, tuple(layers))

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "retention":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
                if m.rot_dims:
                    mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            elif layer.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.temp_coef:
                    mixer["q_temp"] = {"coef": m.temp_coef, "every": m.temp_every}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": layers}

    def model_spec(self) -> ModelSpec:
        blocks = []
        W, eps = self.width, self.norm_eps
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer.mixer
            names = {r: p + "mix." + r for r in ("q", "k", "v", "o")}
            names["gate"] = p + "mix.g"
            if layer.type == "retention":
                rope = RopeSpec(rotary_dim=m.rot_dims, theta=m.rot_base, pairing="half") if m.rot_dims else None
                mixer = RetentionSpec(hidden_size=W, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, decay=m.decay,
                                      key_scale=m.dim ** -0.5, eps=eps, position=rope, weights=names)
            elif layer.type == "attention":
                names.update(q_norm=p + "mix.q.norm", k_norm=p + "mix.k.norm", head_bias=p + "mix.pb")
                mixer = SigmoidAttentionSpec(
                    hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                    scale=m.scale, eps=eps, qk_norm=True, temperature_coef=m.temp_coef, temperature_every=m.temp_every,
                    slope_exponent=SLOPE_EXPONENT, head_bias=True, gated=True, weights=names)
            else:
                names = {"q": p + "mix.q", "down": p + "mix.dkv", "down_norm": p + "mix.dkv.norm", "up_k": p + "mix.uk",
                         "up_v": p + "mix.uv", "gate": p + "mix.g", "o": p + "mix.o"}
                mixer = LatentAttentionSpec(hidden_size=W, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim,
                                            latent_dim=m.kv_rank, scale=m.scale, eps=eps, gated=True, weights=names)
            gates = {"mixer_gate": p + "rg1", "mixer_gate_bias": p + "rg1.b"}
            feed_forward = feed_forward_norm = None
            if layer.ff is not None:
                feed_forward = DenseFeedForwardSpec(W, layer.ff, "xielu",
                                                    {"up": p + "mlp.up", "down": p + "mlp.down", "act": p + "mlp.act"})
                feed_forward_norm = NormSpec(W, eps, {"weight": p + "norm2"})
                gates.update(feed_forward_gate=p + "rg2", feed_forward_gate_bias=p + "rg2.b")
            blocks.append(GatedResidualBlockSpec(mixer=mixer, feed_forward=feed_forward,
                                                 mixer_norm=NormSpec(W, eps, {"weight": p + "norm1"}),
                                                 feed_forward_norm=feed_forward_norm, weights=gates))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=W,
            max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, W, 1.0, {"weight": "embed"}),
            layers=tuple(blocks),
            schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            final_norm=NormSpec(W, eps, {"weight": "final.norm"}),
            head=HeadSpec(self.vocab, W, True, {}, logit_scale=self.logit_scale),
        )
