"""Lovurax without a GPU: the configuration reader, the plain implementation against cases worked out by hand, the
cache and state a model of the design asks for, and a random model folder read back by name."""

import copy
import math

import pytest
import torch

from plain import plain_lovurax as pl
from tiny_lovurax import LVX, attention, latent, retention

F = torch.float64


def test_the_configuration_reads_every_constant_and_round_trips():
    from models_b200.config import config_from_dict

    for raw in LVX.values():
        config = config_from_dict(raw)
        assert config_from_dict(config.to_dict()) == config
        spec = config.model_spec()
        assert spec.head.tied and spec.head.logit_scale == raw["logit_scale"]
        for layer, block in zip(raw["layers"], spec.layers):
            m = layer["mixer"]
            assert (block.feed_forward is None) == (layer["mlp"] is None) == (block.feed_forward_norm is None)
            assert ("feed_forward_gate" in block.weights) == (layer["mlp"] is not None)
            if layer["type"] == "retention":
                assert block.mixer.kind == "retention" and block.mixer.decay == tuple(m["decay"])
                assert block.mixer.key_scale == m["dim"] ** -0.5
                assert (block.mixer.position is None) == ("rot" not in m)
                if "rot" in m:
                    assert (block.mixer.position.rotary_dim, block.mixer.position.theta) == (m["rot"]["dims"], m["rot"]["base"])
            elif layer["type"] == "attention":
                assert block.mixer.kind == "sigmoid_attention" and block.mixer.scale == m["scale"]
                temp = m.get("q_temp") or {"coef": 0.0, "every": 1}
                assert (block.mixer.temperature_coef, block.mixer.temperature_every) == (temp["coef"], temp["every"])
                assert block.mixer.slope_exponent == 8.0
            else:
                assert block.mixer.kind == "latent_attention" and block.mixer.latent_dim == m["kv_rank"]


def test_the_configuration_names_what_is_wrong():
    from models_b200.config import ConfigError, config_from_dict

    raw = copy.deepcopy(LVX["A"])
    raw["layers"][0]["mixer"]["decay"] = [0.5]
    with pytest.raises(ConfigError, match="decay"):
        config_from_dict(raw)
    raw = copy.deepcopy(LVX["A"])
    raw["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="kv_heads"):
        config_from_dict(raw)
    raw = copy.deepcopy(LVX["A"])
    raw["layers"][2]["type"] = "convolution"
    with pytest.raises(ConfigError, match="not built"):
        config_from_dict(raw)
    raw = copy.deepcopy(LVX["A"])
    raw["layers"][0]["mixer"]["rot"]["dims"] = 18
    with pytest.raises(ConfigError, match="rot.dims"):
        config_from_dict(raw)
    raw = copy.deepcopy(LVX["A"])
    del raw["layers"][2]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        config_from_dict(raw)
    raw = copy.deepcopy(LVX["A"])
    raw["layers"][1]["mixer"]["q_temp"]["every"] = 0
    with pytest.raises(ConfigError, match="every"):
        config_from_dict(raw)


def test_xielu_by_hand():
    p, q = torch.tensor(0.0, dtype=F), torch.tensor(0.0, dtype=F)  # softplus(0) = ln 2
    z = torch.tensor([2.0, 0.0, -1.0], dtype=F)
    want = [math.log(2.0) * 4.0 + 1.0, 0.0, (0.5 + math.log(2.0)) * (math.exp(-1.0) - 1.0 + 1.0) - 0.5]
    assert torch.allclose(pl.xielu(z, p, q), torch.tensor(want, dtype=F), atol=1e-12)


def test_rotation_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=F)  # dims 4: pairs (1, 3) and (2, 4); the fifth passes
    out = pl.rotate_half(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0),
            4 * math.cos(a1) + 2 * math.sin(a1), 5.0]
    assert torch.allclose(out[0, 0], torch.tensor(want, dtype=F), atol=1e-12)


def test_the_recurrence_and_its_sums_agree_and_carry_over():
    gen = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(40, n, generator=gen, dtype=F) for n in (6, 6, 9))
    for decay in (0.0, 0.7, 1.0):
        whole, last = pl.retention_states(q, k, v, decay)
        assert torch.allclose(whole, pl.retention_sums(q, k, v, decay), atol=1e-10)
        first, state = pl.retention_states(q[:13], k[:13], v[:13], decay)
        rest, state = pl.retention_states(q[13:], k[13:], v[13:], decay, state)
        assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-12) and torch.allclose(state, last, atol=1e-12)
    # decay 0 keeps the newest token only: o_t = (q_t . k_t) v_t
    assert torch.allclose(pl.retention_states(q, k, v, 0.0)[0], (q * k).sum(1, keepdim=True) * v, atol=1e-12)


def test_sigmoid_attention_by_hand():
    """One head, two tokens, unit matrices: the weights are sigmoids of the scores, each on its own."""
    w = {"q": torch.eye(2, dtype=F), "k": torch.eye(2, dtype=F), "v": torch.eye(2, dtype=F), "g": torch.zeros(2, 2, dtype=F),
         "o": torch.eye(2, dtype=F), "q.norm": torch.ones(2, dtype=F), "k.norm": torch.ones(2, dtype=F), "pb": torch.tensor([0.25], dtype=F)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.5, "q_temp": {"coef": 2.0, "every": 2}}
    h = torch.tensor([[3.0, 4.0], [4.0, 3.0]], dtype=F)
    out = pl.sigmoid_attention(h, w, m, 0.0)
    n = h / math.sqrt(12.5)  # rows divided by their root mean square
    temp1 = 1.0 + 2.0 * math.log(2.0)  # position 1: floor(2 / 2) + 1 = 2; position 0: floor(1 / 2) + 1 = 1
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    w00 = sig(0.5 * float(n[0] @ n[0]) + 0.25)
    w10 = sig(0.5 * temp1 * float(n[1] @ n[0]) - 2.0 ** -8 + 0.25)
    w11 = sig(0.5 * temp1 * float(n[1] @ n[1]) + 0.25)
    want = torch.stack([w00 * h[0], w10 * h[0] + w11 * h[1]]) * 0.5  # the gate is sigmoid(0)
    assert torch.allclose(out, want, atol=1e-12)


def test_latent_attention_equals_attention_in_the_latent_space():
    """Scores and results written with expanded keys and values equal those taken through the latent rows."""
    gen = torch.Generator().manual_seed(2)
    H, D, Dv, R, W, T = 3, 5, 7, 11, 13, 9
    w = {"q": torch.randn(H * D, W, generator=gen, dtype=F), "dkv": torch.randn(R, W, generator=gen, dtype=F),
         "dkv.norm": torch.rand(R, generator=gen, dtype=F) + 0.5, "uk": torch.randn(H * D, R, generator=gen, dtype=F),
         "uv": torch.randn(H * Dv, R, generator=gen, dtype=F), "g": torch.randn(H, W, generator=gen, dtype=F),
         "o": torch.randn(W, H * Dv, generator=gen, dtype=F)}
    m = {"heads": H, "dim": D, "vdim": Dv, "kv_rank": R, "scale": 0.3}
    h = torch.randn(T, W, generator=gen, dtype=F)
    out = pl.latent_attention(h, w, m, 1e-6)
    c = pl.rms_norm(h @ w["dkv"].T, w["dkv.norm"], 1e-6)
    heads = []
    for head in range(H):
        q_latent = (h @ w["q"].T)[:, head * D:(head + 1) * D] @ w["uk"][head * D:(head + 1) * D]
        score = torch.where(torch.ones(T, T).tril().bool(), 0.3 * q_latent @ c.T, torch.full((), -math.inf, dtype=F))
        mixed = torch.softmax(score, -1) @ c
        heads.append(mixed @ w["uv"][head * Dv:(head + 1) * Dv].T * pl.sigmoid(h @ w["g"][head])[:, None])
    assert torch.allclose(out, torch.cat(heads, dim=1) @ w["o"].T, atol=1e-9)


def test_the_cache_and_state_a_model_asks_for():
    """Attention layers of equal shape share a cache group, a latent layer keeps one row per position and no values,
    a retention layer keeps no pages and a float32 state [heads, dim, vdim] per sequence."""
    from models_b200.cache import KvCache, StateArea
    from models_b200.config import config_from_dict
    from models_b200.engine.model import DecoderModel
    from models_b200.parts import Runtime

    raw = {"architecture": "Lovurax", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
           "layers": [attention(2, 1, 8, 16, 0.3, (0.5, 4), 40), retention(2, 8, 4, [0.5, 0.9], (4, 100.0), None),
                      attention(2, 1, 8, 16, 0.2, None, 40), latent(2, 8, 8, 24, 0.3, 40)]}
    model = DecoderModel(config_from_dict(raw).model_spec(), Runtime(torch.device("meta"), "float32", max_positions=1))
    requests = model.kv_requests()
    assert requests[1] is None and requests[0] == requests[2]
    assert (requests[3].num_kv_heads, requests[3].head_dim, requests[3].value_head_dim) == (1, 24, 0)
    cache = KvCache(requests, [None] * 4, max_tokens=256, max_slots=3)
    assert [g.runs for g in cache.groups] == [[0, 2], [3]]
    shapes = []
    cache.allocate_storage(lambda shape: shapes.append(shape))
    assert shapes == [(2, 5, 1, 64, 8), (2, 5, 1, 64, 16), (1, 5, 1, 64, 24), (1, 5, 1, 64, 0)]
    states = model.state_requests()
    assert [s is not None for s in states] == [False, True, False, False] and states[1].shape == (2, 8, 4)
    area = StateArea(states, 3, lambda shape, dtype: torch.ones(shape, dtype=dtype))
    assert area.of_run(1).shape == (4, 2, 8, 4) and area.of_run(0) is None
    area.reset(1)
    assert float(area.of_run(1)[1].abs().sum()) == 0.0 and float(area.of_run(1)[0].sum()) == 64.0


def test_random_model_folder_loads_by_name_and_reports_what_is_wrong(tmp_path):
    import json

    from models_b200.config import load_config
    from models_b200.engine.model import parameter_requests
    from models_b200.weights import WeightsError, load_tensors
    from tiny_lovurax import make_folder

    folder = make_folder(LVX["B"], 5, tmp_path)
    requests = parameter_requests(load_config(folder).model_spec())
    tensors = load_tensors(folder, requests)
    assert set(tensors) == set(requests)
    assert tensors["l0.mix.dkv.norm"].shape == (40,) and tensors["l2.mix.pb"].shape == (3,) and tensors["l1.mlp.act"].shape == (2,)
    assert "l0.norm2" not in tensors and "l0.rg2" not in tensors and "l1.rg2.b" in tensors  # the first layer has no feed-forward
    assert "head" not in tensors  # the output reuses the embedding table
    logits = pl.forward(*pl.read_model_folder(folder), [1, 2, 3, 4, 5])
    assert logits.shape == (5, LVX["B"]["vocab"]) and bool(torch.isfinite(logits).all())
    raw = json.loads((folder / "config.json").read_text())
    raw["layers"][2]["mixer"]["heads"] = 6
    (folder / "config.json").write_text(json.dumps(raw))
    with pytest.raises(WeightsError, match="l2.mix.pb"):
        load_tensors(folder, parameter_requests(load_config(folder).model_spec()))
