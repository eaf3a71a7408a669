"""Small Lovurax configurations for the tests.  They differ from one another in every size and constant, and between
their own layers: the order of the mixers, head counts (also one head, one key/value head, as many key/value heads as
heads), key and value sizes (equal, unequal, no multiples of 8), rotation of part of a head, of a whole head and none,
decays of 1 and below (a decay of 0 makes a head's result the sign of one dot product, which no
bfloat16 comparison survives: the kernel's own test has it), temperature periods shorter than a cache page, layers without a feed-forward, a logit
scale of 1, and widths the tensor-core products do not take."""

from __future__ import annotations

from pathlib import Path

import torch

from plain import plain_lovurax


def retention(heads, dim, vdim, decay, rot, ff):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "retention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def attention(heads, kv_heads, dim, vdim, scale, temp, ff):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if temp is not None:
        mixer["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent(heads, dim, vdim, rank, scale, ff):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


LVX_A = {
    "architecture": "Lovurax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
    "layers": [retention(2, 16, 24, [0.9, 0.995], (8, 10000.0), 96),
               attention(4, 2, 16, 8, 0.25, (0.3, 16), None),
               latent(2, 12, 20, 24, 0.3, 80),
               attention(2, 2, 24, 24, 0.2, (0.7, 50), 72)],
}

LVX_B = {
    "architecture": "Lovurax", "vocab": 150, "width": 72, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
    "layers": [latent(3, 8, 8, 40, 0.35, None),
               retention(1, 32, 32, [1.0], (32, 500.0), 100),
               attention(3, 1, 20, 12, 0.22, (1.0, 5), 50),
               retention(3, 10, 6, [0.5, 0.25, 0.99], None, None),
               attention(1, 1, 8, 40, 0.35, None, 24)],
}

# sizes at which the tensor-core products run (multiples of 64 and more than 128 rows in a prompt)
LVX_C = {
    "architecture": "Lovurax", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [attention(8, 2, 64, 64, 0.125, (0.4, 64), 512),
               latent(4, 64, 64, 128, 0.125, 256),
               retention(4, 64, 128, [0.97, 0.99, 0.999, 0.9], (32, 100000.0), 512)],
}

# a width and head sizes that are no multiples of 8: no tensor-core product or attention takes them
LVX_D = {
    "architecture": "Lovurax", "vocab": 131, "width": 50, "norm": {"eps": 3e-6}, "logit_scale": 0.7,
    "layers": [attention(3, 1, 18, 7, 0.22, (0.9, 3), 77),
               latent(3, 10, 6, 22, 0.3, None),
               retention(2, 18, 10, [0.9, 0.97], (6, 3000.0), 33),
               attention(6, 3, 16, 16, 0.2, None, 40)],
}

LVX = {"A": LVX_A, "B": LVX_B, "C": LVX_C, "D": LVX_D}


def make_folder(raw: dict, seed: int, root, std: float = 0.15) -> Path:
    from models_b200.config import config_from_dict
    from models_b200.weights import write_random_model

    folder = Path(root) / f"lovurax_{seed}"
    write_random_model(folder, config_from_dict(raw), seed, std=std, gain_std=0.1, dtype=torch.bfloat16)
    return folder


def plain_logits(folder, tokens, hidden_out=None) -> torch.Tensor:
    config, weights = plain_lovurax.read_model_folder(folder)
    return plain_lovurax.forward(config, weights, list(tokens), hidden_out)
