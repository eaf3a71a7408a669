"""Small Kabanex configurations for the tests.  They differ from one another in every size and constant,
and between their own layers: head counts (also one head, and as many key/value heads as heads), key and
value sizes (equal, unequal, no multiples of 8), partial and whole-head rotation, windows shorter and
longer than a cache page, kept first positions (none, fewer and more than the window), layers without a
feed-forward, widths the tensor-core products do not take."""

from __future__ import annotations

from pathlib import Path

import torch

from plain import plain_kabanex


def _layer(heads, kv_heads, dim, vdim, rot_dims, base, window, keep_first, scale, recurrent, ff, left_scale, right_scale):
    return {
        "type": "parallel",
        "mixer": {
            "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                     "rot": {"dims": rot_dims, "base": base}, "mask": {"size": window, "keep_first": keep_first}},
            "right": {"width": recurrent}, "left_scale": left_scale, "right_scale": right_scale,
        },
        "mlp": None if ff is None else {"kind": "dense", "ff": ff},
    }


KBX_A = {
    "architecture": "Kabanex", "vocab": 200, "width": 64, "norm": {"eps": 1e-5},
    "layers": [_layer(4, 2, 16, 32, 8, 10000.0, 12, 3, 0.25, 48, 96, 0.7, 1.3),
               _layer(4, 2, 16, 32, 8, 10000.0, 12, 3, 0.25, 48, 96, 0.7, 1.3)],
}

KBX_B = {
    "architecture": "Kabanex", "vocab": 150, "width": 72, "norm": {"eps": 1e-6},
    "layers": [_layer(3, 3, 24, 24, 24, 500.0, 70, 0, 0.2, 40, None, 1.0, 1.0),
               _layer(4, 1, 20, 12, 10, 100000.0, 5, 9, 0.3, 56, 100, 1.5, 0.25),
               _layer(1, 1, 32, 8, 2, 77.0, 1, 2, 0.15, 8, 24, 0.9, 2.0)],
}

KBX_C = {
    "architecture": "Kabanex", "vocab": 131, "width": 50, "norm": {"eps": 3e-6},
    "layers": [_layer(2, 1, 18, 10, 6, 3000.0, 33, 1, 0.22, 30, 77, 1.1, 0.6),
               _layer(2, 2, 18, 10, 18, 3000.0, 64, 5, 0.22, 30, None, 0.8, 0.9)],
}

# sizes at which the tensor-core products run (multiples of 64 and more than 128 rows in a prompt)
KBX_D = {
    "architecture": "Kabanex", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
    "layers": [_layer(4, 2, 64, 128, 32, 10000.0, 100, 2, 0.125, 192, 512, 1.0, 0.5),
               _layer(8, 8, 32, 32, 32, 10000.0, 130, 0, 0.17, 128, 256, 0.5, 1.0)],
}

KBX = {"A": KBX_A, "B": KBX_B, "C": KBX_C, "D": KBX_D}


def make_folder(raw: dict, seed: int, root, std: float = 0.15) -> Path:
    from models_b200.config import config_from_dict
    from models_b200.weights import write_random_model

    folder = Path(root) / f"kabanex_{seed}"
    write_random_model(folder, config_from_dict(raw), seed, std=std, gain_std=0.1, dtype=torch.bfloat16)
    return folder


def plain_logits(folder, tokens, hidden_out=None) -> torch.Tensor:
    config, weights = plain_kabanex.read_model_folder(folder)
    return plain_kabanex.forward(config, weights, list(tokens), hidden_out)
