"""The plain Kabanex implementation against cases worked out by hand, the configuration reader, and the
cache's bookkeeping for windows that keep the first positions.  No GPU."""

import math

import pytest
import torch

from plain import plain_kabanex as pk
from tiny_kabanex import KBX

F = torch.float64


def test_layer_norm_by_hand():
    x = torch.tensor([[1.0, 3.0]], dtype=F)  # mean 2, deviations -1 and 1, variance 1
    out = pk.layer_norm(x, torch.tensor([2.0, 4.0], dtype=F), torch.tensor([0.5, -0.5], dtype=F), 3.0)
    assert torch.allclose(out, torch.tensor([[-1.0 / 2.0 * 2.0 + 0.5, 1.0 / 2.0 * 4.0 - 0.5]], dtype=F))


def test_rotation_pairs_the_halves_of_the_rotated_part_only():
    t = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F).repeat(2, 1, 1)  # dims 4: pairs (0, 2) and (1, 3)
    out = pk.rotate(t, torch.tensor([0, 3]), 4, 100.0)
    assert torch.equal(out[0], t[0])  # position 0 turns nothing
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    expect = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
              3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(out[1, 0], torch.tensor(expect, dtype=F))


def test_visibility_window_and_kept_first_positions():
    m = pk.visible(8, 3, 2)
    assert m[7].tolist() == [True, True, False, False, False, True, True, True]
    assert m[2].tolist() == [True, True, True, False, False, False, False, False]
    assert pk.visible(4, None, 0)[3].tolist() == [True] * 4
    assert pk.visible(5, 1, 0)[4].tolist() == [False, False, False, False, True]


def test_weights_are_mixed_after_the_softmax_and_values_stay_with_their_own_head():
    # two heads, one key/value head each; head 0 looks at key 0 only, head 1 at key 1 only (huge scores)
    big = 50.0
    q = torch.tensor([[[0.0], [0.0]], [[big], [-big]]], dtype=F)  # [T=2, H=2, D=1]
    k = torch.tensor([[[-1.0], [-1.0]], [[0.0], [0.0]]], dtype=F)
    v = torch.tensor([[[1.0], [10.0]], [[2.0], [20.0]]], dtype=F)
    talk = torch.tensor([[1.0, 0.5], [-1.0, 2.0]], dtype=F)
    out = pk.talking_attention(q, k, v, talk, None, 1.0, None, 0)
    # token 1: head 0 -> key 1 (score 0 against -50), head 1 -> key 0 (score 50 against 0)
    # mixed head 0 = 1 * w0 + 0.5 * w1 = [0.5, 1.0] on head 0's values (1, 2); head 1 = -w0 + 2 w1 = [2, -1] on (10, 20)
    assert torch.allclose(out[1, :, 0], torch.tensor([0.5 * 1 + 1.0 * 2, 2 * 10 - 1 * 20], dtype=F), atol=1e-9)
    gated = pk.talking_attention(q, k, v, talk, torch.zeros((2, 2), dtype=F), 1.0, None, 0)
    assert torch.allclose(gated, out * 0.5)


def test_min_gru_by_hand():
    z_in = torch.tensor([[0.0], [0.0]], dtype=F)  # z = 1/2
    x_in = torch.tensor([[1.0], [-30.0]], dtype=F)  # candidates 1.5 and sigmoid(-30) ~ 0
    states = pk.min_gru(z_in, x_in)
    assert torch.allclose(states[:, 0], torch.tensor([0.75, 0.375], dtype=F), atol=1e-12)
    carried = pk.min_gru(z_in[1:], x_in[1:], start=states[0])
    assert torch.allclose(carried[0], states[1])


def test_feed_forward_is_relu_squared():
    h = torch.tensor([[1.0, -1.0]], dtype=F)
    up = torch.tensor([[2.0, 0.0], [0.0, 3.0]], dtype=F)  # up.h = (2, -3) -> relu^2 = (4, 0)
    down = torch.tensor([[1.0, 1.0], [0.5, 7.0]], dtype=F)
    assert torch.allclose(pk.dense_feed_forward(h, up, down), torch.tensor([[4.0, 2.0]], dtype=F))


@pytest.mark.parametrize("name", sorted(KBX))
def test_configuration_round_trip_and_tensor_list(name):
    from models_b200.config import KabanexConfig, config_from_dict
    from models_b200.engine.model import parameter_requests

    raw = KBX[name]
    config = config_from_dict(raw)
    assert isinstance(config, KabanexConfig) and config.to_dict() == raw
    spec = config.model_spec()
    requests = parameter_requests(spec)
    layer = raw["layers"][-1]
    last = len(raw["layers"]) - 1
    left = layer["mixer"]["left"]
    assert tuple(requests[f"l{last}.mix.left.v"].shape) == (left["kv_heads"] * left["vdim"], raw["width"])
    assert tuple(requests[f"l{last}.mix.left.talk"].shape) == (left["heads"], left["heads"])
    assert tuple(requests[f"l{last}.mix.right.x.b"].shape) == (layer["mixer"]["right"]["width"],)
    assert (f"l{last}.mlp.up" in requests) == (layer["mlp"] is not None)
    assert tuple(requests["final.norm.b"].shape) == (raw["width"],)


def test_configuration_errors_name_the_key():
    from models_b200.config import ConfigError, config_from_dict

    import copy
    raw = copy.deepcopy(KBX["A"])
    raw["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="multiple of kv_heads"):
        config_from_dict(raw)
    raw = copy.deepcopy(KBX["A"])
    del raw["layers"][0]["mixer"]["right_scale"]
    with pytest.raises(ConfigError, match="right_scale"):
        config_from_dict(raw)
    raw = copy.deepcopy(KBX["A"])
    raw["layers"][0]["type"] = "serial"
    with pytest.raises(ConfigError, match="not built"):
        config_from_dict(raw)


def test_a_window_group_keeps_the_pages_of_the_first_positions():
    from models_b200.cache.kv_cache import KvCache, KvRequest

    cache = KvCache([KvRequest(1, 8, window=10, value_dim=4, keep_first=3), KvRequest(1, 8, window=10)], [None, None],
                    max_tokens=64 * 16, max_slots=2)
    assert len(cache.groups) == 2  # kept positions make another group: its pages live longer
    slot = cache.open_slot()
    for _ in range(5):
        cache.append([(slot, 64)])
        cache.commit([(slot, 64)])
    keeps, drops = cache.groups[0].tables[slot], cache.groups[1].tables[slot]
    assert keeps[0] >= 0 and all(p < 0 for p in keeps[1:4]) and keeps[4] >= 0
    assert all(p < 0 for p in drops[:4]) and drops[4] >= 0
    cache.check()
    cache.release(slot)
    cache.check()
    assert cache.groups[0].pages.held == 0


def test_random_model_folder_loads_by_name_and_reports_what_is_wrong(tmp_path):
    """The random-weights mode writes a Kabanex folder that the loader reads back tensor by tensor; a folder whose
    talk matrix has another head count is refused with the tensor's name."""
    import json

    from models_b200.config import load_config
    from models_b200.engine.model import parameter_requests
    from models_b200.weights import WeightsError, load_tensors
    from tiny_kabanex import make_folder

    folder = make_folder(KBX["B"], 5, tmp_path)
    config = load_config(folder)
    requests = parameter_requests(config.model_spec())
    tensors = load_tensors(folder, requests)
    assert set(tensors) == set(requests)
    assert tensors["l1.mix.left.talk"].shape == (4, 4) and tensors["l1.mix.right.z.b"].dtype == torch.bfloat16
    assert "l0.mlp.up" not in tensors and "l1.mlp.up" in tensors  # the first layer has no feed-forward
    logits = pk.forward(*pk.read_model_folder(folder), [1, 2, 3, 4, 5])
    assert logits.shape == (5, KBX["B"]["vocab"]) and bool(torch.isfinite(logits).all())
    raw = json.loads((folder / "config.json").read_text())
    raw["layers"][1]["mixer"]["left"]["heads"] = 8
    (folder / "config.json").write_text(json.dumps(raw))
    with pytest.raises(WeightsError, match="l1.mix.left.talk"):
        load_tensors(folder, parameter_requests(load_config(folder).model_spec()))
