"""The Lovurax decoder in the engine against the plain implementation (tests/plain/plain_lovurax.py): each kernel alone
with inputs made so that one key, one position or one state entry decides the result, whole prompts, prompts cut into
portions, token-by-token decoding across cache pages and temperature periods, unequal batches, slots, pages and states
used again, long decoding from CUDA graphs, and greedy generation through the public entry point."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from plain import plain_lovurax as pl
from tiny import TOLERANCE, random_tokens, scaled_error
from tiny_lovurax import LVX, make_folder, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
F = torch.float64


def _engine(folder, dtype, max_tokens=2048, **more):
    from models_b200.engine.loading import engine_from_folder

    return engine_from_folder(folder, dtype, max_tokens, **more)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("lovurax")
    return {name: make_folder(raw, seed=71 + i, root=root) for i, (name, raw) in enumerate(LVX.items())}


def _tolerance(name, dtype):
    """Largest allowed scaled error of logits.  Retention divides a head's result by its root mean square, so the first
    tokens of a sequence, whose results are sums of one or a few dot products, pass the SIGN and relative size of small
    numbers on at full scale: in bfloat16 the configuration with two retention layers and a narrow width shows about
    twice the error of the others (float32 is held to the common bound everywhere)."""
    return 2 * TOLERANCE[dtype] if (name, dtype) == ("B", "bfloat16") else TOLERANCE[dtype]


def _rounded(t, dtype):
    return t.to(dtype).to(F)


# ----------------------------------------------------------------------------------- kernels alone

def _pools(T, G, D, Dv, page_size, device, dtype, shuffle_seed=0):
    """Fresh pools with the sequence's pages in a shuffled order: pools, page table, slot mapping, positions."""
    pages = -(-T // page_size)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(shuffle_seed)) + 1
    k_pool = torch.full((pages + 1, G, page_size, D), float("nan"), dtype=dtype, device=device)
    v_pool = torch.full((pages + 1, G, page_size, Dv), float("nan"), dtype=dtype, device=device) if Dv else None
    positions = torch.arange(T, dtype=torch.int32)
    mapping = (order[positions // page_size].to(torch.int32) * page_size + positions % page_size).to(torch.int32).to(device)
    return k_pool, v_pool, order.to(torch.int32)[None, :].contiguous().to(device), mapping, positions.to(device)


def _sigmoid_attend(q, k, v, gains, temp, bias, gate, scale, dtype, device, page_size=64, q_len=None, kernel=None):
    """norm_store then the sigmoid attention for the last `q_len` tokens of one sequence: float64 [q_len, H * Dv]."""
    from models_b200.kernels import ops

    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    q_len = T if q_len is None else q_len
    k_pool, v_pool, table, mapping, positions = _pools(T, G, D, Dv, page_size, device, dtype)
    wide = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(dtype).to(device)
    a, b = H * D, H * D + G * D
    qg, kg = (None, None) if gains is None else (gains[0].float().to(device), gains[1].float().to(device))
    ops.norm_store(wide[:, :a], wide[:, a:b], wide[:, b:], positions, qg, kg, 1e-6, temp[0], temp[1], k_pool, v_pool, mapping,
                   H, G, D, Dv)
    out = torch.empty((q_len, H * Dv), dtype=dtype, device=device)
    cu_q = torch.tensor([0, q_len], dtype=torch.int32, device=device)
    kv_lens = torch.tensor([T], dtype=torch.int32, device=device)
    ops.gated_attention(wide[T - q_len:, :a], out, k_pool, v_pool, table, cu_q, kv_lens, q_len, H, G, D, Dv, "sigmoid", scale, 8.0,
                        bias.float().to(device) if bias is not None else None,
                        gate[T - q_len:].to(dtype).to(device).contiguous() if gate is not None else None,
                        "element" if gate is not None else None, kernel)
    return out.double().cpu()


def _plain_sigmoid_attend(q, k, v, gains, temp, bias, gate, scale):
    T, H, D = q.shape
    G = k.shape[1]
    if gains is not None:
        q, k = pl.rms_norm(q, gains[0].to(F), 1e-6), pl.rms_norm(k, gains[1].to(F), 1e-6)
    pos = torch.arange(T)
    if temp[0]:
        q = q * (1.0 + temp[0] * torch.log(torch.floor((pos + 1).to(F) / temp[1]) + 1.0))[:, None, None]
    distance = (pos[:, None] - pos[None, :]).to(F)
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        score = (q[:, h] @ k[:, h // (H // G)].T) * scale - 2.0 ** (-8.0 * (h + 1) / H) * distance + (bias[h] if bias is not None else 0.0)
        out[:, h] = torch.where(distance >= 0, pl.sigmoid(score), torch.zeros((), dtype=F)) @ v[:, h // (H // G)]
    out = out.reshape(T, -1)
    return out * pl.sigmoid(gate.to(F)) if gate is not None else out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,target", [(700, 3), (700, 0), (130, 63), (130, 64), (65, 64), (321, 255), (40, 39)])
def test_one_key_decides_the_sigmoid_attention(cuda_device, tokens, target, dtype):
    """All keys but one score far below zero (weights near 0); the key at `target` -- far back among hundreds, the
    first position, either side of a page border, the query's own position -- scores near zero, where the distance
    term and the head's bias move the weight, and carries a value found nowhere else."""
    H, G, D, Dv = 4, 2, 16, 16
    gen = torch.Generator().manual_seed(tokens * 1000 + target)
    direction = torch.nn.functional.normalize(torch.randn(D, generator=gen, dtype=F), dim=0)
    q = torch.randn(tokens, H, D, generator=gen, dtype=F) * 0.1
    k = torch.randn(tokens, G, D, generator=gen, dtype=F) * 0.1 - 6.0 * direction
    q[-1] += 6.0 * direction
    # the flattest head's score of the target comes out near 1/2: its distance term is made up for in the key
    k[target] += (6.0 + (2.0 ** -8 * (tokens - 1 - target) - 0.5) / 6.0) * direction
    v = torch.randn(tokens, G, Dv, generator=gen, dtype=F) * 0.01
    v[target] += 5.0
    bias = torch.tensor([0.5, -0.25, 0.0, 1.0], dtype=F)
    q, k, v = _rounded(q, dtype), _rounded(k, dtype), _rounded(v, dtype)
    want = _plain_sigmoid_attend(q, k, v, None, (0.0, 1), bias, None, 1.0)[-1:]
    weight = want.reshape(H, Dv).mean(1) / 5.0  # (the steeper heads' weights of a far key are next to nothing)
    assert 0.05 < float(weight[-1]) < 0.95  # the flattest head's weight of the target is in the sigmoid's sensitive range
    for kernel in ("decode", "rows") + (("tc",) if dtype == torch.bfloat16 else ()):  # one token is a (short) prompt step too
        got = _sigmoid_attend(q, k, v, None, (0.0, 1), bias, None, 1.0, dtype, cuda_device, q_len=1, kernel=kernel)
        assert scaled_error(got, want) < (2e-5 if dtype == torch.float32 else 2e-2), kernel


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,every", [(1, 1, 8, 8, 32, 1), (6, 2, 20, 12, 64, 7), (3, 3, 40, 72, 128, 64),
                                                                 (16, 4, 64, 160, 64, 33), (4, 1, 128, 300, 64, 1000)])
def test_sigmoid_attention_sizes_norm_temperature_and_gate(cuda_device, heads, kv_heads, dim, vdim, page, every, dtype):
    """Prompt rows and a decoded row at sizes that are equal, 1, and no multiples of 8; the temperature's period is
    passed many times, once, or never."""
    T = 150
    gen = torch.Generator().manual_seed(heads * 100 + dim)
    q = _rounded(torch.randn(T, heads, dim, generator=gen, dtype=F), dtype)
    k = _rounded(torch.randn(T, kv_heads, dim, generator=gen, dtype=F), dtype)
    v = _rounded(torch.randn(T, kv_heads, vdim, generator=gen, dtype=F), dtype)
    gains = (1.0 + 0.3 * torch.randn(dim, generator=gen), 1.0 + 0.3 * torch.randn(dim, generator=gen))
    gate = _rounded(torch.randn(T, heads * vdim, generator=gen, dtype=F), dtype)
    bias = torch.randn(heads, generator=gen).to(F) - 2.0
    want = _plain_sigmoid_attend(q, k, v, gains, (0.6, every), bias, gate, 0.3)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for q_len, kernel in ((T, None), (1, None), (37, None), (T, "rows"), (1, "rows")):
        # (None: the tensor-core form for bfloat16 prompts of sizes it takes, the split-key form for one token)
        got = _sigmoid_attend(q, k, v, gains, (0.6, every), bias, gate, 0.3, dtype, cuda_device, page_size=page, q_len=q_len, kernel=kernel)
        assert scaled_error(got, want[T - q_len:]) < tol, (q_len, kernel)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_temperature_steps_exactly_at_its_period(cuda_device, dtype):
    """Queries at positions period - 2, period - 1, period (p + 1 just below, at and above a multiple) with equal
    contents: the stored query changes by exactly the temperature's step, and only where floor((p + 1) / period) does."""
    from models_b200.kernels import ops

    period, coef, D = 48, 0.9, 16
    T = 3 * period
    row = torch.randn(D, dtype=F)
    q = _rounded(row.repeat(T, 1), dtype).to(dtype).to(cuda_device)
    k = q.clone()
    k_pool, _, _, mapping, positions = _pools(T, 1, D, 0, 64, cuda_device, dtype)
    ops.norm_store(q, k, None, positions, None, None, 1e-6, coef, period, k_pool, None, mapping, 1, 1, D, 0)
    factor = (q.double().cpu() / _rounded(row, dtype)[None, :]).mean(1)
    expected = torch.tensor([1.0 + coef * math.log((p + 1) // period + 1) for p in range(T)], dtype=F)
    assert scaled_error(factor, expected) < (1e-6 if dtype == torch.float32 else 6e-3)
    assert float(factor[period - 2]) == pytest.approx(1.0, abs=1e-6 if dtype == torch.float32 else 6e-3)
    assert float(factor[period - 1]) == pytest.approx(1.0 + coef * math.log(2.0), rel=1e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,target", [(600, 5), (129, 63), (129, 64), (64, 0), (300, 299)])
def test_one_latent_row_decides_the_softmax(cuda_device, tokens, target, dtype):
    """The cache holds one row per position, read as key and as value; one row -- far back among hundreds, at a page
    border, the first, the query's own -- has the largest score by a wide margin, so the result is that row."""
    from models_b200.kernels import ops

    H, R = 3, 40
    gen = torch.Generator().manual_seed(tokens + target)
    rows = _rounded(torch.randn(tokens, 1, R, generator=gen, dtype=F), dtype)
    q = torch.randn(1, H, R, generator=gen, dtype=F) * 0.05
    q += 1.5 * rows[target, 0][None, None, :] / rows[target, 0].norm() * torch.tensor([1.0, 2.0, 3.0], dtype=F)[None, :, None]
    q = _rounded(q, dtype)
    k_pool, _, table, mapping, positions = _pools(tokens, 1, R, 0, 64, cuda_device, dtype, shuffle_seed=3)
    ops.norm_store(None, rows.reshape(tokens, R).to(dtype).to(cuda_device), None, positions, None, None, 1e-6, 0.0, 1, k_pool, None,
                   mapping, 0, 1, R, 0)
    out = torch.empty((1, H * R), dtype=dtype, device=cuda_device)
    cu_q = torch.tensor([0, 1], dtype=torch.int32, device=cuda_device)
    kv_lens = torch.tensor([tokens], dtype=torch.int32, device=cuda_device)
    ops.gated_attention(q.reshape(1, -1).to(dtype).to(cuda_device), out, k_pool, None, table, cu_q, kv_lens, 1, H, 1, R, R, "softmax", 2.0)
    weights = torch.softmax(2.0 * (q[0] @ rows[:, 0].T), dim=-1)
    assert float(weights[-1, target]) > 0.9
    want = (weights @ rows[:, 0]).reshape(1, -1)
    assert scaled_error(out, want) < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,tokens", [(5, 48, 200), (16, 256, 330), (2, 40, 70), (9, 64, 129)])
def test_softmax_over_shared_rows_in_every_form(cuda_device, heads, rank, tokens, dtype):
    """All heads read the same cached rows as keys and as values; prompts (the tensor-core form where it takes the
    sizes), a portion of a prompt, and one token with the keys cut into runs; a gate per head."""
    from models_b200.kernels import ops

    gen = torch.Generator().manual_seed(rank + tokens)
    rows = _rounded(torch.randn(tokens, rank, generator=gen, dtype=F), dtype)
    q = _rounded(torch.randn(tokens, heads, rank, generator=gen, dtype=F) * 0.5, dtype)
    gate = _rounded(torch.randn(tokens, heads, generator=gen, dtype=F), dtype)
    k_pool, _, table, mapping, positions = _pools(tokens, 1, rank, 0, 64, cuda_device, dtype, shuffle_seed=5)
    ops.norm_store(None, rows.to(dtype).to(cuda_device), None, positions, None, None, 1e-6, 0.0, 1, k_pool, None, mapping, 0, 1, rank, 0)
    visible = torch.ones(tokens, tokens).tril().bool()
    want = []
    for h in range(heads):
        score = torch.where(visible, 0.2 * q[:, h] @ rows.T, torch.full((), -math.inf, dtype=F))
        want.append(torch.softmax(score, -1) @ rows * pl.sigmoid(gate[:, h:h + 1]))
    want = torch.stack(want, dim=1).reshape(tokens, -1)
    kv_lens = torch.tensor([tokens], dtype=torch.int32, device=cuda_device)
    for q_len, kernel in ((tokens, None), (33, None), (1, None), (tokens, "rows"), (1, "rows")):
        out = torch.empty((q_len, heads * rank), dtype=dtype, device=cuda_device)
        cu_q = torch.tensor([0, q_len], dtype=torch.int32, device=cuda_device)
        ops.gated_attention(q[tokens - q_len:].reshape(q_len, -1).to(dtype).to(cuda_device), out, k_pool, None, table, cu_q, kv_lens, q_len,
                            heads, 1, rank, rank, "softmax", 0.2, 0.0, None, gate[tokens - q_len:].to(dtype).to(cuda_device).contiguous(),
                            "head", kernel)
        assert scaled_error(out, want[tokens - q_len:]) < (2e-5 if dtype == torch.float32 else 2e-2), (q_len, kernel)


def test_decode_runs_cover_the_page_table():
    from models_b200.kernels import ops

    for sequences, heads, kv_heads, pages in ((1, 4, 2, 1), (1, 16, 1, 512), (8, 16, 4, 24), (64, 32, 8, 3), (2, 3, 3, 100)):
        runs, span = ops.gated_decode_runs(sequences, heads, kv_heads, pages)
        assert runs >= 1 and span >= 1 and runs * span >= pages and (runs - 1) * span < pages and runs <= 64


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,n_in,n_out,tokens", [(1, 8, 8, 1), (3, 12, 40, 17), (5, 40, 6, 100), (4, 64, 128, 33), (2, 256, 80, 200),
                                                     (3, 48, 256, 64)])
def test_one_small_matrix_per_head(cuda_device, heads, n_in, n_out, tokens, dtype):
    from models_b200.kernels import ops

    gen = torch.Generator().manual_seed(n_in)
    x = _rounded(torch.randn(tokens, heads, n_in, generator=gen, dtype=F), dtype)
    w = _rounded(torch.randn(heads, n_out, n_in, generator=gen, dtype=F), dtype)
    gate = _rounded(torch.randn(tokens, heads, generator=gen, dtype=F), dtype)
    wide = torch.zeros((tokens, heads * n_in + 8), dtype=dtype, device=cuda_device)  # a column slice of a wider tensor
    wide[:, 8:] = x.reshape(tokens, -1).to(dtype)
    out = torch.empty((tokens, heads * n_out), dtype=dtype, device=cuda_device)
    for g in (None, gate):
        for tensor_cores in (True, False):  # (the tensor-core form takes the last case's bfloat16 run)
            ops.head_linear(wide[:, 8:], w.to(dtype).to(cuda_device), out, heads, g.to(dtype).to(cuda_device) if g is not None else None,
                            tensor_cores)
            want = torch.einsum("thk,hnk->thn", x, w)
            if g is not None:
                want = want * pl.sigmoid(g)[:, :, None]
            assert scaled_error(out, want.reshape(tokens, -1)) < (1e-5 if dtype == torch.float32 else 1e-2), tensor_cores


def _plain_retention(q, k, v, g, decay, rot, first_position, eps, start=None):
    """One sequence's new tokens from the state `start` [H, D, Dv]: results [T, H * Dv] and the new state."""
    T, H, D = q.shape
    pos = torch.arange(first_position, first_position + T)
    q = pl.rotate_half(q, pos, rot[0], rot[1], torch.float32)
    k = pl.rotate_half(k, pos, rot[0], rot[1], torch.float32) * D ** -0.5
    outs, states = [], []
    for h in range(H):
        o, S = pl.retention_states(q[:, h], k[:, h], v[:, h], decay[h], None if start is None else start[h])
        outs.append(o)
        states.append(S)
    o = pl.rms_norm(torch.stack(outs, dim=1), None, eps).reshape(T, -1)
    return o * (g * pl.sigmoid(g)), torch.stack(states)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("run_length", [0, 16, 7])
@pytest.mark.parametrize("heads,dim,vdim,rot,decay", [(2, 16, 24, (8, 10000.0), [0.9, 0.999]), (1, 32, 32, (32, 50.0), [1.0]),
                                                      (3, 10, 6, (0, 1.0), [0.5, 0.0, 0.97]), (2, 64, 128, (48, 2e5), [0.99, 0.95]),
                                                      (2, 32, 7, (16, 300.0), [0.9, 0.8]), (1, 128, 256, (64, 1e4), [0.98])])
def test_retention_ragged_carried_and_rotated(cuda_device, heads, dim, vdim, rot, decay, run_length, dtype):
    """Sequences of unequal lengths in one call, then one more token for each (the state is carried in float32 between
    calls, positions go on from where the sequence stands, far from zero for one of them), rows of unused slots
    untouched; decays of 0 (no memory), 1 (nothing forgotten) and in between; the sequences walked whole, and in runs of
    16 and of 7 tokens at once (the last run of a sequence is shorter, some sequences have one run, some runs are empty)."""
    from models_b200.kernels import ops
    from models_b200.parts.rope import RotaryEmbedding
    from models_b200.config.specs import RopeSpec
    from models_b200.parts import Runtime

    device = cuda_device
    lengths, starts = [1, 9, 70, 33], [0, 0, 1000, 5]
    gen = torch.Generator().manual_seed(dim + vdim)
    tables = RotaryEmbedding(RopeSpec(rot[0], rot[1], "half"), Runtime(device, "float32", max_positions=1200)) if rot[0] else None
    slots_total = 6
    state = torch.zeros((slots_total + 1, heads, dim, vdim), dtype=torch.float32, device=device)
    state[5] = 7.0  # an unused slot: must stay as it is
    slots = torch.tensor([4, 0, 2, 1], dtype=torch.int32, device=device)
    plain_state = [None] * 4
    # the third sequence stands at position 1000 with a state of its own
    carried = torch.randn(heads, dim, vdim, generator=gen, dtype=torch.float32)
    state[2] = carried.to(device)
    plain_state[2] = carried.to(F)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for call in range(3):
        counts = lengths if call == 0 else [1, 1, 1, 1]
        total = sum(counts)
        width = 2 * heads * dim + 2 * heads * vdim
        proj = _rounded(torch.randn(total, width, generator=gen, dtype=F), dtype)
        a, b, c = heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim
        dev = proj.to(dtype).to(device)
        cu = [0]
        for n in counts:
            cu.append(cu[-1] + n)
        positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, counts)]).to(torch.int32).to(device)
        out = torch.empty((total, heads * vdim), dtype=dtype, device=device)
        ops.retention_scan(dev[:, :a], dev[:, a:b], dev[:, b:c], dev[:, c:], positions, tables.cos if tables else None,
                           tables.sin if tables else None, rot[0], torch.tensor(decay, dtype=torch.float32, device=device),
                           dim ** -0.5, 1e-6, state, slots, torch.tensor(cu, dtype=torch.int32, device=device), heads, dim, vdim, out,
                           1.0, max(counts), run_length)
        for i, n in enumerate(counts):
            rows = proj[cu[i]:cu[i + 1]]
            want, plain_state[i] = _plain_retention(rows[:, :a].view(n, heads, dim), rows[:, a:b].view(n, heads, dim),
                                                    rows[:, b:c].view(n, heads, vdim), rows[:, c:], decay, rot, starts[i], 1e-6,
                                                    plain_state[i])
            assert scaled_error(out[cu[i]:cu[i + 1]], want) < tol, (call, i)
            assert scaled_error(state[int(slots[i])], plain_state[i]) < 1e-5, (call, i)
            starts[i] += n
    assert bool((state[5] == 7.0).all()) and bool((state[3] == 0.0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_retention_remembers_one_far_token(cuda_device, dtype):
    """A decay of exactly 1 and keys that are zero but for one far token: hundreds of steps later the query that matches
    that key reads that token's value, undamped; with a decay below 1 it reads it damped by decay^distance."""
    from models_b200.kernels import ops

    device, T, D, Dv, far = cuda_device, 400, 8, 16, 7
    q = torch.zeros(T, 2 * D)
    k = torch.zeros(T, 2 * D)
    k[far, 3] = k[far, D + 3] = 2.0
    q[-1, 3] = q[-1, D + 3] = 1.5
    v = torch.randn(T, 2 * Dv)
    g = torch.ones(T, 2 * Dv)
    proj = torch.cat([q, k, v, g], dim=1).to(dtype).to(device)
    state = torch.zeros((2, 2, D, Dv), dtype=torch.float32, device=device)
    out = torch.empty((T, 2 * Dv), dtype=dtype, device=device)
    decay = [1.0, 0.99]
    ops.retention_scan(proj[:, :2 * D], proj[:, 2 * D:4 * D], proj[:, 4 * D:4 * D + 2 * Dv], proj[:, 4 * D + 2 * Dv:],
                       torch.arange(T, dtype=torch.int32, device=device), None, None, 0, torch.tensor(decay, device=device), 1.0, 1e-30,
                       state, torch.tensor([0], dtype=torch.int32, device=device), torch.tensor([0, T], dtype=torch.int32, device=device),
                       2, D, Dv, out)
    value = proj[far, 4 * D:4 * D + 2 * Dv].double().cpu().view(2, Dv)
    silu = 1.0 / (1.0 + math.exp(-1.0))
    want = torch.cat([value[h] / value[h].pow(2).mean().sqrt() * silu for h in range(2)])  # the norm takes the damping out again
    assert scaled_error(out[-1], want) < (1e-5 if dtype == torch.float32 else 1e-2)
    S = state[0].double().cpu()
    assert scaled_error(S[0, 3], 2.0 * value[0]) < 1e-6
    assert scaled_error(S[1, 3], 2.0 * value[1] * 0.99 ** (T - 1 - far)) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_xielu_and_the_gated_residual_add(cuda_device, dtype):
    from models_b200.kernels import ops

    gen = torch.Generator().manual_seed(5)
    z = _rounded(torch.randn(33, 72, generator=gen, dtype=F) * 3.0, dtype)
    p, q = torch.tensor(0.3, dtype=F), torch.tensor(-0.7, dtype=F)
    wide = torch.zeros((33, 96), dtype=dtype, device=cuda_device)
    ops.xielu(z.to(dtype).to(cuda_device), wide[:, 8:80], float(pl.softplus(p)), float(0.5 + pl.softplus(q)))
    assert scaled_error(wide[:, 8:80], pl.xielu(z, p, q)) < (1e-6 if dtype == torch.float32 else 5e-3)
    assert bool((wide[:, :8] == 0).all()) and bool((wide[:, 80:] == 0).all())
    x = torch.randn(33, 72, generator=gen)
    gate = _rounded(torch.randn(33, 72, generator=gen, dtype=F) * 2.0, dtype)
    bias = torch.randn(72, generator=gen)
    delta = torch.randn(33, 72, generator=gen)
    wide[:, 8:80] = gate.to(dtype)
    got = ops.gated_residual_add(x.to(cuda_device), wide[:, 8:80], bias.to(cuda_device), delta.to(cuda_device))
    assert scaled_error(got, x.to(F) + pl.sigmoid(gate + bias.to(F)) * delta.to(F)) < 1e-6


@pytest.mark.parametrize("rows,n,k", [(1, 64, 128), (8, 72, 200), (5, 256, 1024)])
def test_the_gated_add_rides_in_the_last_product_of_a_decode_step(cuda_device, rows, n, k):
    """x += sigmoid(gate + bias) * (a . W^T) by the decode product's epilogue against the same in float64."""
    from models_b200.kernels import ops

    gen = torch.Generator().manual_seed(rows + n)
    a = torch.randn(rows, k, generator=gen).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=gen) * 0.1).to(torch.bfloat16)
    x = torch.randn(rows, n, generator=gen)
    wide = torch.randn(rows, n + 16, generator=gen).to(torch.bfloat16)  # the gate is a column slice
    bias = torch.randn(n, generator=gen)
    want = x.to(F) + pl.sigmoid(wide[:, 8:8 + n].to(F) + bias.to(F)) * (a.to(F) @ w.to(F).T)
    got = x.to(cuda_device)
    ops.skinny_gemm_gated_residual(w.to(cuda_device), a.to(cuda_device), got, wide.to(cuda_device)[:, 8:8 + n], bias.to(cuda_device))
    assert scaled_error(got, want) < 2e-5


# ----------------------------------------------------------------------------------- the model in the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(LVX))
def test_whole_prompt_every_position(cuda_device, folders, name, dtype):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    for n, seed in ((1, 1), (7, 2), (70, 3), (200, 4)):
        tokens = random_tokens(LVX[name]["vocab"], n, seed)
        slot = engine.open_slot()
        logits = engine.step([StepEntry(slot, tokens, list(range(n)))])
        engine.release_slot(slot)
        assert scaled_error(logits, plain_logits(folders[name], tokens)) < _tolerance(name, dtype), (name, dtype, n)
    engine.cache.check()


@pytest.mark.parametrize("name", sorted(LVX))
def test_residual_stream_after_every_layer(cuda_device, folders, name):
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], "float32")
    tokens = random_tokens(LVX[name]["vocab"], 90, 6)
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
@pytest.mark.parametrize("name", sorted(LVX))
def test_prompt_then_token_by_token(cuda_device, folders, name, dtype):
    """A short prompt, then 130 tokens one by one: the decode path crosses cache pages and many periods of the query
    temperature, and the retention state is carried through every step."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    n, head = 150, 20
    tokens = random_tokens(LVX[name]["vocab"], n, 7)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, tokens[:head], [head - 1])])]
    for i in range(head, n):
        rows.append(engine.step([StepEntry(slot, [tokens[i]], [0])]))
    got = torch.cat(rows)
    assert scaled_error(got, expected[head - 1:]) < _tolerance(name, dtype)
    engine.cache.check()
    engine.release_slot(slot)
    assert all(g.pages.held == 0 for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,portions", [("A", [2, 3, 17, 64, 1, 2, 90, 21]), ("B", [64, 64, 2, 70]), ("C", [130, 2, 68]),
                                           ("D", [5, 2, 2, 129, 62])])
def test_prompt_in_portions(cuda_device, folders, name, portions, dtype):
    """A portion starts inside a sequence: its recurrence goes on from the stored state, its queries see the keys and
    latent rows of earlier portions, and its positions (rotation, temperature, distances) go on from where it stands."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype)
    tokens = random_tokens(LVX[name]["vocab"], sum(portions), 8)
    expected = plain_logits(folders[name], tokens)
    slot = engine.open_slot()
    at = 0
    for count in portions:
        got = engine.step([StepEntry(slot, tokens[at:at + count], list(range(count)))])
        assert scaled_error(got, expected[at:at + count]) < _tolerance(name, dtype), (at, count)
        at += count


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(LVX))
def test_unequal_batches_and_slots_used_again(cuda_device, folders, name, dtype):
    """Four prompts of unequal lengths in one step, decoded together while the shorter ones end; then new requests take
    the freed slots and pages (their states must start at zero, their pages hold old keys)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=1024)
    vocab = LVX[name]["vocab"]
    tol = _tolerance(name, dtype)
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
    """Three sequences decoded for 330 steps from captured steps, over several pages; one sequence ends on the way and
    another takes its slot (and must not inherit its state)."""
    from models_b200.engine import StepEntry

    engine = _engine(folders[name], dtype, max_tokens=4096)
    engine.enable_decode_graphs(4)
    vocab = LVX[name]["vocab"]
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
    assert worst < _tolerance(name, dtype)
    assert engine.decode_graphs.captured  # the steps did come from captures
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["retention", "attention", "latent"])
def test_models_of_one_kind_of_layer(cuda_device, tmp_path, kind, dtype):
    """Only retention layers (no cache group at all, state alone), only attention or only latent layers (no state, so
    prompt steps are replayed from captures from their third occurrence on): prompts of one length class four times
    over, then tokens one by one from captured decode steps."""
    from models_b200.engine import StepEntry
    from tiny_lovurax import attention, latent, retention

    layers = {"retention": [retention(2, 16, 24, [0.9, 0.99], (8, 1e4), 48), retention(1, 32, 16, [0.95], None, None)],
              "attention": [attention(4, 2, 16, 8, 0.25, (0.3, 16), 48), attention(2, 1, 32, 32, 0.2, None, None)],
              "latent": [latent(2, 12, 20, 24, 0.3, 48), latent(4, 16, 16, 32, 0.25, None)]}[kind]
    raw = {"architecture": "Lovurax", "vocab": 120, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.3, "layers": layers}
    folder = make_folder(raw, 90, tmp_path)
    engine = _engine(folder, dtype, 1024)
    engine.enable_decode_graphs(4)
    assert (engine.prompt_graphs is None) == (kind == "retention") and (len(engine.cache.groups) == 0) == (kind == "retention")
    for seed in range(4):
        tokens = random_tokens(120, 140, seed)
        want = plain_logits(folder, tokens)
        slot = engine.open_slot()
        rows = [engine.step([StepEntry(slot, tokens[:100], [99])])]
        for t in tokens[100:]:
            rows.append(engine.decode([slot], [t]).clone())
        assert scaled_error(torch.cat(rows), want[99:]) < TOLERANCE[dtype], seed
        engine.release_slot(slot)
    engine.cache.check()


def test_logits_do_not_depend_on_the_batch_or_the_cut(cuda_device, folders):
    """float32: the same position through a whole prompt, through portions, and inside a batch differs by rounding only."""
    from models_b200.engine import StepEntry

    engine = _engine(folders["A"], "float32")
    vocab = LVX["A"]["vocab"]
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
    prompts = [random_tokens(LVX["A"]["vocab"], n, 50 + n) for n in (3, 40, 11)]
    steps = 40
    config, weights = pl.read_model_folder(folder)
    expected, margins = [], []
    for prompt in prompts:
        tokens, out, margin = list(prompt), [], []
        for _ in range(steps):
            logits = pl.forward(config, weights, tokens)[-1]
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
    """bin/trace_run on a Lovurax folder: two prompts in one step, then decoded together from captured steps."""
    name = "B"
    vocab = LVX[name]["vocab"]
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
                               "--out", str(out), "--max-tokens", "102"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        ea, eb = plain_logits(folders[name], a), plain_logits(folders[name], b)
        first = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, vocab)
        tol = _tolerance(name, dtype)
        assert scaled_error(first[0], ea[0]) < tol and scaled_error(first[1], ea[69]) < tol and scaled_error(first[2], eb[4]) < tol
        for i in range(20):
            got = np.fromfile(out / f"{i + 1}.f32", dtype="<f4").reshape(-1, vocab)
            assert scaled_error(got[0], ea[70 + i]) < tol, i
            if i < 7:
                assert scaled_error(got[1], eb[5 + i]) < tol, i
