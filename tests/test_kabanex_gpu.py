"""The Kabanex decoder in the engine against the plain implementation (tests/plain/plain_kabanex.py):
each kernel alone with inputs made so that one key decides the result, whole prompts, prompts cut into
portions, token-by-token decoding across windows and cache pages, unequal batches, slots and pages used
again, long decoding from CUDA graphs, and greedy generation through the public entry point."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from plain import plain_kabanex as pk
from tiny import TOLERANCE, random_tokens, scaled_error
from tiny_kabanex import KBX, make_folder, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
F = torch.float64


def _engine(folder, dtype, max_tokens=2048, **more):
    from models_b200.engine.loading import engine_from_folder

    return engine_from_folder(folder, dtype, max_tokens, **more)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("kabanex")
    return {name: make_folder(raw, seed=41 + i, root=root) for i, (name, raw) in enumerate(KBX.items())}


# ----------------------------------------------------------------------------------- kernels alone

def _paged(k, v, page_size, device, dtype, shuffle_seed=0):
    """Stores k [T, G, D] and v [T, G, Dv] in fresh pools through the rotate-and-store kernel (no rotation), with
    the sequence's pages in a shuffled order.  Returns pools, page table, slot mapping."""
    from models_b200.kernels import ops

    T, G, D = k.shape
    Dv = v.shape[2]
    pages = -(-T // page_size)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(shuffle_seed)) + 1
    k_pool = torch.zeros((pages + 1, G, page_size, D), dtype=dtype, device=device)
    v_pool = torch.full((pages + 1, G, page_size, Dv), float("nan"), dtype=dtype, device=device)
    positions = torch.arange(T, dtype=torch.int32)
    mapping = (order[positions // page_size].to(torch.int32) * page_size + positions % page_size).to(torch.int32).to(device)
    return k_pool, v_pool, order.to(torch.int32)[None, :].contiguous().to(device), mapping, positions.to(device)


def _attend(q, k, v, talk, gate, scale, window, keep_first, dtype, device, page_size=64, q_len=None, out_scale=1.0, kernel=None):
    """The kernel's result for the last `q_len` tokens (all by default) of one sequence, as float64 [q_len, H, Dv]."""
    from models_b200.kernels import ops

    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    q_len = T if q_len is None else q_len
    k_pool, v_pool, table, mapping, positions = _paged(k, v, page_size, device, dtype)
    wide = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(dtype).to(device)
    a, b = H * D, H * D + G * D
    ops.rotate_store(wide[:, :a], wide[:, a:b], wide[:, b:], positions, None, None, k_pool, v_pool, mapping, H, G, D, Dv, 0)
    rows = wide[T - q_len:]
    out = torch.empty((q_len, H * Dv), dtype=dtype, device=device)
    cu_q = torch.tensor([0, q_len], dtype=torch.int32, device=device)
    kv_lens = torch.tensor([T], dtype=torch.int32, device=device)
    gate_d = gate[T - q_len:].to(dtype).to(device).contiguous() if gate is not None else None
    talk_d = talk.float().to(device).contiguous() if talk is not None else None
    ops.talking_attention(rows[:, :a], out, k_pool, v_pool, table, cu_q, kv_lens, q_len, H, G, D, Dv, window, keep_first, scale,
                          talk_d, gate_d, out_scale, kernel)
    return out.double().cpu().reshape(q_len, H, Dv)


def _rounded(t, dtype):
    return t.to(dtype).to(F)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,window,keep_first,target", [
    (200, 45, 6, 155),   # the oldest key of the window
    (200, 45, 6, 154),   # the first key outside it
    (200, 45, 6, 5),     # the last kept first position
    (200, 45, 6, 6),     # the first position that is not kept
    (200, 45, 0, 0),     # nothing kept: position 0 is gone
    (200, 70, 2, 130),   # window longer than a page: its oldest key
    (200, 70, 2, 129),
    (130, 3, 9, 8),      # more kept positions than the window is long
    (130, 3, 9, 9),
    (700, None, 0, 0),   # no window: the first key among 700
    (700, None, 0, 63),  # the last position of the first page
    (700, None, 0, 64),  # the first position of the second page
    (321, 1, 1, 320),    # a window of the query's own position
    (321, 1, 1, 319),
])
def test_one_key_decides_the_attention(cuda_device, tokens, window, keep_first, target, dtype):
    """The last query's heads all point at one key, whose value is far from the others'.  Whether that key is
    visible changes the result grossly; every row is compared with the plain attention."""
    g = torch.Generator().manual_seed(tokens + target)
    H, G, D, Dv = 4, 2, 16, 16
    q = torch.randn((tokens, H, D), generator=g, dtype=F)
    k = torch.randn((tokens, G, D), generator=g, dtype=F)
    v = torch.randn((tokens, G, Dv), generator=g, dtype=F)
    talk = torch.randn((H, H), generator=g, dtype=F)
    gate = torch.randn((tokens, H), generator=g, dtype=F)
    direction = torch.zeros(D, dtype=F)
    direction[5] = 8.0
    q[-1] = direction  # score 64 * scale with the target, about 8 * scale * N(0, 1) with every other key
    k[target] = direction
    v[target] = 100.0
    q, k, v, gate = (_rounded(t, dtype) for t in (q, k, v, gate))
    expected = pk.talking_attention(q, k, v, talk.float().to(F), gate, 0.5, window, keep_first)
    seen = pk.visible(tokens, window, keep_first)[-1, target].item()
    assert (expected[-1].abs().max() > 10.0) == seen  # the case shows what it is meant to show
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for kernel in ("rows", "tc") if dtype == torch.bfloat16 else ("rows",):  # a block per token; the tensor-core tiles
        got = _attend(q, k, v, talk, gate, 0.5, window, keep_first, dtype, cuda_device, kernel=kernel)
        assert scaled_error(got, expected) < tol, kernel
        part = _attend(q, k, v, talk, gate, 0.5, window, keep_first, dtype, cuda_device, q_len=37, kernel=kernel)  # a portion
        assert scaled_error(part, expected[-37:]) < tol, kernel
    for kernel in ("decode", "rows"):  # as a decode step sees it: the keys' chunks with a block each; a block for the token
        last = _attend(q, k, v, talk, gate, 0.5, window, keep_first, dtype, cuda_device, q_len=1, kernel=kernel)
        assert scaled_error(last[0], expected[-1]) < tol, kernel


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page", [(1, 1, 8, 8, 32), (6, 2, 20, 12, 64), (3, 3, 40, 72, 128), (16, 4, 64, 128, 64),
                                                          (1, 1, 16, 16, 32), (6, 2, 80, 160, 64), (8, 8, 32, 48, 128), (12, 2, 48, 64, 64)])
def test_attention_sizes_mixing_gate_and_scale(cuda_device, heads, kv_heads, dim, vdim, page, dtype):
    g = torch.Generator().manual_seed(heads * 100 + dim)
    T = 150
    q, k = torch.randn((T, heads, dim), generator=g, dtype=F), torch.randn((T, kv_heads, dim), generator=g, dtype=F)
    v = torch.randn((T, kv_heads, vdim), generator=g, dtype=F)
    talk = torch.randn((heads, heads), generator=g, dtype=F)
    gate = torch.randn((T, heads), generator=g, dtype=F)
    q, k, v, gate = (_rounded(t, dtype) for t in (q, k, v, gate))
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for use_talk, use_gate, out_scale in ((True, True, 1.7), (False, True, 1.0), (True, False, 0.5)):
        expected = out_scale * pk.talking_attention(q, k, v, talk.float().to(F) if use_talk else None, gate if use_gate else None,
                                                    0.3, 37, 5)
        takes_tc = dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0
        for kernel in ("rows", "tc") if takes_tc else ("rows",):
            got = _attend(q, k, v, talk if use_talk else None, gate if use_gate else None, 0.3, 37, 5, dtype, cuda_device,
                          page_size=page, out_scale=out_scale, kernel=kernel)
            assert scaled_error(got, expected) < tol, (use_talk, use_gate, kernel)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_of_part_of_a_head_and_the_cache_write(cuda_device, dtype):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(5)
    T, H, G, D, Dv, dims, base = 70, 3, 1, 20, 6, 12, 300.0
    q, k, v = (_rounded(torch.randn(s, generator=g, dtype=F), dtype) for s in ((T, H, D), (T, G, D), (T, G, Dv)))
    positions = torch.arange(1000, 1000 + T)
    angle = positions.to(F)[:, None] * torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)[None, :]
    cos = torch.zeros((1000 + T, dims // 2), dtype=torch.float32)
    sin = torch.zeros_like(cos)
    cos[1000:], sin[1000:] = torch.cos(angle).float(), torch.sin(angle).float()
    k_pool, v_pool, table, mapping, _ = _paged(k, v, 32, cuda_device, dtype)
    wide = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(dtype).to(cuda_device)
    a, b = H * D, H * D + G * D
    ops.rotate_store(wide[:, :a], wide[:, a:b], wide[:, b:], positions.to(torch.int32).to(cuda_device), cos.to(cuda_device),
                     sin.to(cuda_device), k_pool, v_pool, mapping, H, G, D, Dv, dims)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    assert scaled_error(wide[:, :a].double().cpu().reshape(T, H, D), pk.rotate(q, positions, dims, base)) < tol
    flat_k = k_pool.reshape(-1, G, 32, D).permute(0, 2, 1, 3).reshape(-1, G, D)[mapping.cpu().long()]
    flat_v = v_pool.reshape(-1, G, 32, Dv).permute(0, 2, 1, 3).reshape(-1, G, Dv)[mapping.cpu().long()]
    assert scaled_error(flat_k.double().cpu(), pk.rotate(k, positions, dims, base)) < tol
    assert torch.equal(flat_v.double().cpu(), v)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("long_lengths", [[1, 9, 300, 77], [2500, 3, 340, 40]])  # runs of up to 16 tokens; of 20
def test_min_gru_scan_ragged_chunked_and_carried(cuda_device, dtype, long_lengths):
    """Sequences of 1, 9, 300 and 77 new tokens in one call (the long ones are walked in many runs at once), the
    state carried into a second call, a row stride wider than the state, a scale, and gates that nearly freeze
    the state for a while, so that a start lost between runs would show at the end."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(9)
    R, lengths = 45, long_lengths
    total = sum(lengths)
    wide = torch.randn((total, 3 * R + 11), generator=g, dtype=F) * 2.0
    wide[40:330, :R] -= 9.0  # z ~ 1e-4: the state barely moves over hundreds of tokens (they lie in the longest sequence)
    z_bias, x_bias = torch.randn(R, generator=g, dtype=F), torch.randn(R, generator=g, dtype=F)
    wide = _rounded(wide, dtype)
    dev = wide.to(dtype).to(cuda_device)
    state = torch.zeros((6, R), dtype=torch.float32, device=cuda_device)
    slots = torch.tensor([4, 0, 2, 5], dtype=torch.int32, device=cuda_device)
    cu_q = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=cuda_device)
    out = torch.full((total, R + 3), float("nan"), dtype=dtype, device=cuda_device)
    zb, xb = z_bias.float().to(cuda_device), x_bias.float().to(cuda_device)
    ops.mingru_scan(dev[:, :R], dev[:, R:2 * R], dev[:, 2 * R:3 * R], zb, xb, state, slots, cu_q, max(lengths), out[:, 1:R + 1], 0.5)
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    ends = {}
    for b, (first, n) in enumerate(zip(cu_q.tolist(), lengths)):
        rows = wide[first:first + n]
        states = pk.min_gru(rows[:, :R] + z_bias.float().to(F), rows[:, R:2 * R] + x_bias.float().to(F))
        expected = 0.5 * states * pk.silu(rows[:, 2 * R:3 * R])
        assert scaled_error(out[first:first + n, 1:R + 1], expected) < tol, b
        ends[int(slots[b])] = states[-1]
        assert scaled_error(state[int(slots[b])], states[-1]) < 1e-5
    assert torch.isnan(out[:, 0].float()).all() and torch.isnan(out[:, R + 1:].float()).all()  # nothing beside its columns
    assert float(state[[1, 3]].abs().max()) == 0.0  # nor beside its slots
    # a decode step on top: one token for two of the sequences
    step = _rounded(torch.randn((2, 3 * R), generator=g, dtype=F), dtype)
    dev2 = step.to(dtype).to(cuda_device)
    out2 = torch.empty((2, R), dtype=dtype, device=cuda_device)
    ops.mingru_scan(dev2[:, :R], dev2[:, R:2 * R], dev2[:, 2 * R:], zb, xb, state, torch.tensor([2, 4], dtype=torch.int32, device=cuda_device),
                    torch.tensor([0, 1, 2], dtype=torch.int32, device=cuda_device), 1, out2, 1.0)
    for row, slot in enumerate((2, 4)):
        states = pk.min_gru(step[row:row + 1, :R] + z_bias.float().to(F), step[row:row + 1, R:2 * R] + x_bias.float().to(F), ends[slot])
        assert scaled_error(out2[row], (states * pk.silu(step[row:row + 1, 2 * R:]))[0]) < tol


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_rows_far_from_zero(cuda_device, out_dtype):
    """Rows with a mean a thousand times their spread: a variance taken as mean(x^2) - mean^2 would lose them."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(3)
    for width in (50, 320, 1537):
        x = (torch.randn((9, width), generator=g) + 1000.0).float()
        gain, bias = torch.randn(width, generator=g).float(), torch.randn(width, generator=g).float()
        expected = pk.layer_norm(x.to(F), gain.to(F), bias.to(F), 1e-6)
        got = ops.layernorm(x.to(cuda_device), gain.to(cuda_device), bias.to(cuda_device), 1e-6, out_dtype)
        assert scaled_error(got, expected) < (2e-4 if out_dtype == torch.float32 else 8e-3), width
        rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=cuda_device)
        picked = ops.layernorm(x.to(cuda_device), gain.to(cuda_device), bias.to(cuda_device), 1e-6, out_dtype, rows)
        assert torch.equal(picked, got[[7, 0, 7]])


def test_relu_squared_into_a_column_slice(cuda_device):
    from models_b200.kernels import ops

    src = torch.randn((5, 40), device=cuda_device).to(torch.bfloat16)
    dst = torch.zeros((5, 64), dtype=torch.bfloat16, device=cuda_device)
    ops.activate(src[:, 3:36], dst[:, 8:41], "relu2", 2.0)
    expected = (2.0 * torch.relu(src[:, 3:36].float()) ** 2).to(torch.bfloat16)
    assert torch.equal(dst[:, 8:41], expected) and float(dst[:, :8].abs().max()) == 0 and float(dst[:, 41:].abs().max()) == 0


# ----------------------------------------------------------------------------------- the model in the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(KBX))
def test_whole_prompt_every_position(cuda_device, folders, name, dtype):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    for n, seed in ((1, 1), (7, 2), (70, 3), (200, 4)):
        tokens = random_tokens(KBX[name]["vocab"], n, seed)
        slot = engine.open_slot()
        logits = engine.step([StepEntry(slot, tokens, list(range(n)))])
        engine.release_slot(slot)
        assert scaled_error(logits, plain_logits(folders[name], tokens)) < TOLERANCE[dtype], (name, dtype, n)
    engine.cache.check()


@pytest.mark.parametrize("name", ["B", "D"])
def test_residual_stream_after_every_layer(cuda_device, folders, name):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], "float32")
    tokens = random_tokens(KBX[name]["vocab"], 90, 6)
    seen = []
    engine.model.observer = lambda run, x: seen.append(x.double().cpu())
    slot = engine.open_slot()
    engine.step([StepEntry(slot, tokens, [89])])
    expected = []
    plain_logits(folders[name], tokens, expected)
    assert len(seen) == len(expected)
    for layer, (got, want) in enumerate(zip(seen, expected)):
        assert scaled_error(got, want) < 1e-5, layer


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(KBX))
def test_prompt_then_token_by_token(cuda_device, folders, name, dtype):
    """A short prompt, then 130 tokens one by one: the decode kernels pass every window's edge, the kept first
    positions fall out of the window, and pages of the first layers are given back on the way."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    n, head = 150, 20
    tokens = random_tokens(KBX[name]["vocab"], n, 7)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, tokens[:head], [head - 1])])]
    for i in range(head, n):
        rows.append(engine.step([StepEntry(slot, [tokens[i]], [0])]))
    got = torch.cat(rows)
    assert scaled_error(got, expected[head - 1:]) < TOLERANCE[dtype]
    engine.cache.check()
    engine.release_slot(slot)
    assert all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,portions", [("A", [2, 3, 17, 64, 1, 2, 90, 21]), ("B", [64, 64, 2, 70]), ("C", [5, 2, 2, 129, 62]),
                                           ("D", [130, 2, 68])])
def test_prompt_in_portions(cuda_device, folders, name, portions, dtype):
    """A portion starts inside a sequence: its recurrence goes on from the stored state, its queries see the
    keys of earlier portions, and its positions rotate from where the sequence stands."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    tokens = random_tokens(KBX[name]["vocab"], sum(portions), 8)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    at = 0
    for count in portions:
        got = engine.step([StepEntry(slot, tokens[at:at + count], list(range(count)))])
        assert scaled_error(got, expected[at:at + count]) < TOLERANCE[dtype], (at, count)
        at += count


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_unequal_batches_and_slots_used_again(cuda_device, folders, name, dtype):
    """Four prompts of unequal lengths in one step, decoded together while the shorter ones end; then new
    requests take the freed slots and pages (their states must start at zero, their pages hold old keys)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=1024)
    vocab = KBX[name]["vocab"]
    tol = TOLERANCE[dtype]
    for round_index in range(2):
        lengths, prompts = [1, 33, 140, 70], [1, 20, 131, 66]
        full = [random_tokens(vocab, n + 12, 10 * round_index + i) for i, n in enumerate(lengths)]
        expected = [plain_logits(folders[name], t) for t in full]
        slots = [engine.open_slot() for _ in full]
        out = engine.step([StepEntry(s, t[:p], [0, p - 1]) for s, t, p in zip(slots, full, prompts)])
        for i, p in enumerate(prompts):
            assert scaled_error(out[2 * i], expected[i][0]) < tol and scaled_error(out[2 * i + 1], expected[i][p - 1]) < tol, i
        live = list(range(4))
        at = list(prompts)
        while live:
            out = engine.step([StepEntry(slots[i], [full[i][at[i]]], [0]) for i in live])
            for row, i in enumerate(live):
                assert scaled_error(out[row], expected[i][at[i]]) < tol, (round_index, i, at[i])
                at[i] += 1
            for i in [i for i in live if at[i] == len(full[i])]:
                engine.release_slot(slots[i])
                live.remove(i)
        engine.cache.check()
    assert engine.cache.slots.held == 0 and all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_graphs(cuda_device, folders, name, dtype):
    """Three sequences decoded for 330 steps from captured steps: windows slide over several pages, window
    groups give pages back while the pages of kept first positions stay, and one sequence ends on the way and
    another takes its place."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=4096)
    engine.enable_decode_graphs(4)
    vocab = KBX[name]["vocab"]
    full = [random_tokens(vocab, n, 20 + i) for i, n in enumerate((340, 200, 150, 120))]
    expected = [plain_logits(folders[name], t) for t in full]
    prompts = [5, 70, 1, 30]
    slots = {i: engine.open_slot() for i in range(3)}
    engine.step([StepEntry(slots[i], full[i][:prompts[i]], []) for i in range(3)])
    at = {i: prompts[i] for i in range(3)}
    worst = 0.0
    while at:
        live = sorted(at)
        out = engine.decode([slots[i] for i in live], [full[i][at[i]] for i in live])
        for row, i in enumerate(live):
            if at[i] % 7 == 0 or at[i] > len(full[i]) - 3:
                worst = max(worst, scaled_error(out[row], expected[i][at[i]]))
            at[i] += 1
            if at[i] == len(full[i]):
                engine.release_slot(slots.pop(i))
                del at[i]
                if i == 2:  # a new request in the freed slot, from its prompt
                    slots[3] = engine.open_slot()
                    engine.step([StepEntry(slots[3], full[3][:prompts[3]], [])])
                    at[3] = prompts[3]
    assert worst < TOLERANCE[dtype]
    assert engine.decode_graphs.captured  # the steps did come from captures
    engine.cache.check()


def test_logits_do_not_depend_on_the_batch_or_the_cut(cuda_device, folders):
    """float32: the same position through a whole prompt, through portions, and inside a batch differs by
    rounding only (a few units of the last place of the largest logit)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders["A"], "float32")
    vocab = KBX["A"]["vocab"]
    a, b = random_tokens(vocab, 100, 31), random_tokens(vocab, 37, 32)
    slot = engine.open_slot()
    whole = engine.step([StepEntry(slot, a, [99])])
    engine.release_slot(slot)
    s1, s2 = engine.open_slot(), engine.open_slot()
    engine.step([StepEntry(s2, b[:30], []), StepEntry(s1, a[:64], [])])
    engine.step([StepEntry(s1, a[64:99], []), StepEntry(s2, b[30:], [])])
    cut = engine.step([StepEntry(s1, a[99:], [0])])
    assert scaled_error(cut, whole) < 5e-6


def test_greedy_generation_through_the_entry_point(cuda_device, folders):
    import models_b200

    folder = folders["A"]
    prompts = [random_tokens(KBX["A"]["vocab"], n, 50 + n) for n in (3, 40, 11)]
    steps = 40  # past the window of 12 and the 3 kept positions
    config, weights = pk.read_model_folder(folder)
    expected, margins = [], []
    for prompt in prompts:
        tokens, out, margin = list(prompt), [], []
        for _ in range(steps):
            logits = pk.forward(config, weights, tokens)[-1]
            top = torch.topk(logits, 2).values
            margin.append(float(top[0] - top[1]))
            out.append(int(torch.argmax(logits)))
            tokens.append(out[-1])
        expected.append(out)
        margins.append(margin)
    for dtype in DTYPES:
        model = models_b200.load_model(folder, dtype=dtype, max_batch=4, context=256)
        results = model.generate_batch(prompts, models_b200.SamplingOptions(temperature=0.0, max_tokens=steps))
        for result, want, margin in zip(results, expected, margins):
            for i, (a, b) in enumerate(zip(result.tokens, want)):
                if a != b:
                    assert dtype == "bfloat16" and margin[i] < 0.05, (dtype, i, result.tokens, want)
                    break
        model.close()


def test_trace_replay_program(cuda_device, folders, tmp_path):
    """bin/trace_run on a Kabanex folder: two prompts in one step, then decoded together from captured steps."""
    name = "B"
    vocab = KBX[name]["vocab"]
    a, b = random_tokens(vocab, 90, 1), random_tokens(vocab, 12, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for i in range(20):
        entries = [{"id": "a", "tokens": [a[70 + i]], "want": [0]}]
        if i < 7:
            entries.append({"id": "b", "tokens": [b[5 + i]], "want": [0]})
        steps.append({"step": i + 1, "entries": entries, "end": (["b"] if i == 6 else []) + (["a"] if i == 19 else [])})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in DTYPES:
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "102"],  # the tokens alone: partly filled pages come on top
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        ea, eb = plain_logits(folders[name], a), plain_logits(folders[name], b)
        first = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, vocab)
        tol = TOLERANCE[dtype]
        assert scaled_error(first[0], ea[0]) < tol and scaled_error(first[1], ea[69]) < tol and scaled_error(first[2], eb[4]) < tol
        for i in range(20):
            got = np.fromfile(out / f"{i + 1}.f32", dtype="<f4").reshape(-1, vocab)
            assert scaled_error(got[0], ea[70 + i]) < tol, i
            if i < 7:
                assert scaled_error(got[1], eb[5 + i]) < tol, i
