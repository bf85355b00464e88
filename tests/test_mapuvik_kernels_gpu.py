"""Each new kernel alone against a plain float64 formula, at sizes of its own, with the
inputs arranged so that a fault shows: a window's edge, a page's border, a far key, a state
carried through portions of every size, slots used again."""

from __future__ import annotations

import math

import pytest
import torch

import plain_mapuvik as plain
from ayaka_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def randn(*shape: int, seed: int, scale: float = 1.0) -> torch.Tensor:
    return torch.randn(*shape, generator=gen(seed), dtype=torch.float64) * scale


def close(got: torch.Tensor, want: torch.Tensor, tol: float, label: str = "") -> None:
    got, want = got.double().cpu(), want.double()
    scale = float(want.abs().max()) or 1.0
    error = float((got - want).abs().max()) / scale
    assert math.isfinite(error) and error <= tol, f"{label}: error {error:.3e} of scale"


# ---- norm -------------------------------------------------------------------------------------
@pytest.mark.parametrize("width, groups", [(48, 1), (96, 4), (1000, 5), (4096, 2)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_with_offset_groups_gather_and_gates(width, groups, out_dtype):
    rows = 9
    x, w, g = randn(rows, width, seed=1, scale=3.0), randn(width, seed=2, scale=0.3), \
        randn(rows, width, seed=3, scale=2.0)
    eps = 1e-3
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    xd, wd, gd = x.float().to(DEV), w.float().to(DEV), g.float().to(DEV)

    def grouped(v):
        return plain.rms(v.reshape(rows, groups, -1), eps).reshape(rows, width)

    out = torch.zeros(rows, width, dtype=out_dtype, device=DEV)
    ops.rms_norm(xd, wd, eps, out, weight_offset=1.0, groups=groups)
    close(out, grouped(x) * (1 + w), tol, "offset")
    index = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    part = torch.zeros(3, width, dtype=out_dtype, device=DEV)
    ops.rms_norm(xd, wd, eps, part, groups=groups, rows=index, count=3)
    close(part, (grouped(x) * w)[[7, 0, 3]], tol, "gather")
    ops.rms_norm(xd, wd, eps, out, groups=groups, gate=gd, gate_mode="silu_before")
    close(out, grouped(x * plain.silu(g)) * w, tol, "gate before")
    ops.rms_norm(xd, wd, eps, out, groups=groups, gate=gd, gate_mode="sigmoid_after")
    close(out, grouped(x) * w * torch.sigmoid(g), tol, "gate after")


# ---- rotation ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_turns_the_named_stretch_of_every_head_and_nothing_else(dtype):
    rows, heads, stride, offset, dims, base = 6, 3, 40, 8, 12, 300.0
    x = randn(rows, heads * stride, seed=4)
    positions = torch.tensor([0, 1, 5, 1000, 77777, 3], dtype=torch.int32)
    xd = x.to(dtype).to(DEV)
    want = xd.double().cpu().reshape(rows, heads, stride).clone()
    want[..., offset:offset + dims] = plain.rotate_pairs(
        want[..., offset:offset + dims], positions, dims, base)
    ops.rope(xd, positions.to(DEV), ops.rope_frequencies(dims, base, torch.device(DEV)),
             heads=heads, head_stride=stride, offset=offset)
    close(xd.reshape(rows, heads, stride), want, 2e-6 if dtype == torch.float32 else 8e-3)
    # the other layout: entry i with entry i + dims / 2
    yd = x.float().to(DEV)
    ops.rope(yd, positions.to(DEV), ops.rope_frequencies(dims, base, torch.device(DEV)),
             heads=heads, head_stride=stride, offset=offset, layout="halves")
    stretch = x.reshape(rows, heads, stride)[..., offset:offset + dims]
    shuffled = torch.stack([stretch[..., :dims // 2], stretch[..., dims // 2:]], dim=-1)
    turned = plain.rotate_pairs(shuffled.reshape(rows, heads, dims), positions, dims, base)
    turned = turned.reshape(rows, heads, dims // 2, 2)
    want = x.reshape(rows, heads, stride).clone()
    want[..., offset:offset + dims // 2] = turned[..., 0]
    want[..., offset + dims // 2:offset + dims] = turned[..., 1]
    close(yd.reshape(rows, heads, stride), want, 2e-6)


# ---- the small products per head --------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, heads, inner, outer", [(1, 1, 8, 8), (37, 3, 20, 70),
                                                       (130, 5, 64, 33)])
def test_head_linear_both_orientations_and_the_gate(dtype, rows, heads, inner, outer):
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    a = randn(rows, heads * inner, seed=5).to(dtype)
    stored = randn(heads * outer, inner, seed=6).to(dtype)       # [out, in] per head
    across = randn(heads * inner, outer, seed=7).to(dtype)       # [in, out] per head
    gate = randn(rows, heads * outer, seed=8)
    a64 = a.double().reshape(rows, heads, inner)
    out = torch.zeros(rows, heads * (outer + 3), dtype=dtype, device=DEV)  # padded heads
    ops.head_linear(a.to(DEV), across.to(DEV), out, heads=heads, transposed=True, rows=rows)
    want = torch.einsum("nhi,hij->nhj", a64, across.double().reshape(heads, inner, outer))
    close(out.reshape(rows, heads, outer + 3)[..., :outer], want, tol, "as stored")
    assert float(out.reshape(rows, heads, outer + 3)[..., outer:].abs().max()) == 0.0
    tight = torch.zeros(rows, heads * outer, dtype=dtype, device=DEV)
    ops.head_linear(a.to(DEV), stored.to(DEV), tight, heads=heads, transposed=False, rows=rows,
                    gate=gate.float().to(DEV))
    want = torch.einsum("nhi,hji->nhj", a64, stored.double().reshape(heads, outer, inner))
    want = want * torch.sigmoid(gate.float().double()).reshape(rows, heads, outer)
    close(tight.reshape(rows, heads, outer), want, tol, "transposed with gate")


@pytest.mark.parametrize("rows, heads, inner, outer", [(17, 2, 8, 8), (64, 3, 64, 72),
                                                       (200, 5, 136, 64), (65, 1, 72, 256)])
def test_head_linear_of_prompt_portions_on_the_tensor_cores(rows, heads, inner, outer):
    """bfloat16, more than 16 rows, sizes in 16-byte pieces: both orientations, heads of ``a``
    and of the result wider than what is used (their padding untouched), the gate, row and
    column counts that end inside a tile, an inner size of more than one turn."""
    dtype, pad = torch.bfloat16, 8
    a = randn(rows, heads, inner + pad, seed=15).to(dtype)
    a[..., inner:] = float("nan")  # (never read)
    stored = randn(heads * outer, inner, seed=16).to(dtype)       # [out, in] per head
    across = randn(heads * inner, outer, seed=17).to(dtype)       # [in, out] per head
    gate = randn(rows, heads * outer, seed=18)
    a64 = a.double()[..., :inner]
    flat = a.reshape(rows, heads * (inner + pad)).to(DEV)
    out = torch.full((rows + 1, heads * (outer + pad)), 3.0, dtype=dtype, device=DEV)
    ops.head_linear(flat, across.to(DEV), out, heads=heads, transposed=True, rows=rows,
                    inner=inner)
    want = torch.einsum("nhi,hij->nhj", a64, across.double().reshape(heads, inner, outer))
    got = out[:rows].reshape(rows, heads, outer + pad)
    close(got[..., :outer], want, 1e-2, "as stored")
    assert float((got[..., outer:] - 3.0).abs().max()) == 0.0
    assert float((out[rows] - 3.0).abs().max()) == 0.0
    tight = torch.full((rows + 1, heads * outer), 3.0, dtype=dtype, device=DEV)
    ops.head_linear(flat, stored.to(DEV), tight, heads=heads, transposed=False, rows=rows,
                    gate=gate.float().to(DEV), inner=inner)
    want = torch.einsum("nhi,hji->nhj", a64, stored.double().reshape(heads, outer, inner))
    want = want * torch.sigmoid(gate.float().double()).reshape(rows, heads, outer)
    close(tight[:rows].reshape(rows, heads, outer), want, 1e-2, "transposed with gate")
    assert float((tight[rows] - 3.0).abs().max()) == 0.0


# ---- attention over latent rows ---------------------------------------------------------------
def _paged(rows_of_request: list[torch.Tensor], page: int, dtype, shuffle_seed: int):
    """Scatter each request's rows [T, D] over pages handed out in a shuffled order."""
    width = rows_of_request[0].shape[1]
    need = [-(-t.shape[0] // page) for t in rows_of_request]
    total = sum(need) + 1
    order = (torch.randperm(total - 1, generator=gen(shuffle_seed)) + 1).tolist()
    pages = torch.full((total, 1, page, width), float("nan"), dtype=torch.float64)
    table = torch.zeros(len(need), max(need), dtype=torch.int32)
    for b, rows in enumerate(rows_of_request):
        for index in range(need[b]):
            page_id = order.pop()
            table[b, index] = page_id
            piece = rows[index * page:(index + 1) * page]
            pages[page_id, 0, :piece.shape[0]] = piece
    return pages.to(dtype).to(DEV), table.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, rank, rot, window, page", [
    (3, 24, 8, 13, 8), (5, 40, 0, 0, 16), (2, 70, 6, 64, 16), (9, 128, 32, 33, 32)])
def test_latent_attention_sees_its_window_and_not_a_key_more(dtype, heads, rank, rot, window,
                                                              page):
    """Two keys are made to stand out for every query: the oldest one its window still holds
    and the one just before it. The first must take nearly all the weight, the second none;
    unwritten page slots hold NaN, so a key read from beyond the sequence shows as well."""
    key_dim = rank + rot
    lengths = [1, 2, page, page + 1, 3 * page - 1, 150]
    keys = [randn(t, key_dim, seed=20 + i, scale=0.3) for i, t in enumerate(lengths)]
    direction = randn(key_dim, seed=9)
    direction = direction / direction.norm()
    queries, request_of_row, positions = [], [], []
    for b, t in enumerate(lengths):
        picked = sorted({0, 1, t // 2, t - 2, t - 1} & set(range(t)))
        for p in picked:
            oldest = max(0, p - window + 1) if window else 0
            keys[b][oldest] += 6.0 * direction
            if oldest > 0:
                keys[b][oldest - 1] += 12.0 * direction  # louder still, and out of sight
            queries.append(randn(heads, key_dim, seed=100 * b + p, scale=0.5)
                           + 3.0 * direction)
            request_of_row.append(b)
            positions.append(p)
    keys = [k.to(dtype).double() for k in keys]
    q = torch.stack(queries).to(dtype)
    pages, table = _paged(keys, page, dtype, shuffle_seed=3)
    n, scale = len(positions), 0.7
    out = torch.zeros(n, heads * rank, dtype=dtype, device=DEV)
    ops.latent_attention(q.reshape(n, heads * key_dim).to(DEV), pages, table,
                         torch.tensor(request_of_row, dtype=torch.int32, device=DEV),
                         torch.tensor(positions, dtype=torch.int32, device=DEV), out,
                         num_heads=heads, rank=rank, scale=scale, window=window)
    got = out.double().cpu().reshape(n, heads, rank)
    assert torch.isfinite(got).all()
    for i, (b, p) in enumerate(zip(request_of_row, positions)):
        lo = max(0, p - window + 1) if window else 0
        seen = keys[b][lo:p + 1]
        weights = torch.softmax(scale * q[i].double() @ seen.T, dim=-1)
        close(got[i], weights @ seen[:, :rank], 2e-5 if dtype == torch.float32 else 1.5e-2,
              f"request {b} position {p}")


@pytest.mark.parametrize("dtype, tensor_cores", [(torch.float32, True), (torch.bfloat16, True),
                                                 (torch.bfloat16, False)])
@pytest.mark.parametrize("heads, rank, rot, window, page, splits", [
    (3, 24, 8, 13, 8, 1), (5, 40, 0, 0, 16, 3), (16, 224, 32, 200, 16, 7), (37, 64, 16, 70, 32, 2),
    (2, 250, 6, 0, 16, 32), (2, 20, 2, 0, 16, 2), (20, 130, 30, 90, 16, 5), (1, 16, 0, 3, 8, 2)])
def test_latent_decode_serves_every_head_from_one_fetch(dtype, tensor_cores, heads, rank, rot,
                                                         window, page, splits):
    """Single rows at the ends of sequences of every length around a tile of 32 keys and a
    page, more shares than some rows have tiles, a window's oldest key loud and the key before
    it louder; against the plain softmax, and against the kernel for any step."""
    key_dim = rank + rot
    lengths = [1, 2, 31, 32, 33, 64, 65, 300, page, page + 1]
    keys = [randn(t, key_dim, seed=60 + i, scale=0.3) for i, t in enumerate(lengths)]
    direction = randn(key_dim, seed=10)
    direction = direction / direction.norm()
    queries = []
    for b, t in enumerate(lengths):
        p = t - 1
        oldest = max(0, p - window + 1) if window else 0
        keys[b][oldest] += 6.0 * direction
        if oldest > 0:
            keys[b][oldest - 1] += 12.0 * direction
        queries.append(randn(heads, key_dim, seed=200 + b, scale=0.5) + 3.0 * direction)
    keys = [k.to(dtype).double() for k in keys]
    q = torch.stack(queries).to(dtype)
    pages, table = _paged(keys, page, dtype, shuffle_seed=4)
    n, scale = len(lengths), 0.6
    request_of_row = torch.arange(n, dtype=torch.int32, device=DEV)
    positions = torch.tensor([t - 1 for t in lengths], dtype=torch.int32, device=DEV)
    out = torch.full((n, heads * (rank + 5)), 7.0, dtype=dtype, device=DEV)  # padded heads
    partial = torch.empty(n * heads * splits * (rank + 2), device=DEV)
    ops.set_latent_decode_tensor_cores(tensor_cores)
    try:
        took = ops.latent_decode(q.reshape(n, heads * key_dim).to(DEV), pages, table,
                                 request_of_row, positions, out, partial, num_heads=heads,
                                 rank=rank, scale=scale, window=window, rows=n, splits=splits)
    finally:
        ops.set_latent_decode_tensor_cores(True)
    if key_dim % 8:
        assert not took
        return
    assert took
    got = out.double().cpu().reshape(n, heads, rank + 5)
    assert torch.all(got[..., rank:] == 7.0)
    other = torch.zeros(n, heads * rank, dtype=dtype, device=DEV)
    ops.latent_attention(q.reshape(n, heads * key_dim).to(DEV), pages, table, request_of_row,
                         positions, other, num_heads=heads, rank=rank, scale=scale,
                         window=window)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for b, t in enumerate(lengths):
        lo = max(0, t - window) if window else 0
        seen = keys[b][lo:t]
        weights = torch.softmax(scale * q[b].double() @ seen.T, dim=-1)
        close(got[b, :, :rank], weights @ seen[:, :rank], tol, f"request {b}")
    close(got[..., :rank], other.double().cpu().reshape(n, heads, rank), tol, "both kernels")


# ---- the short convolution --------------------------------------------------------------------
@pytest.mark.parametrize("channels, taps", [(5, 1), (130, 2), (64, 4), (300, 7)])
def test_the_convolution_carries_its_last_inputs_through_any_cut(channels, taps):
    lengths = {0: 23, 1: 9, 2: 1}
    slots = {0: 2, 1: 0, 2: 3}
    u = {b: randn(t, channels, seed=30 + b) for b, t in lengths.items()}
    weight, bias = randn(channels, taps, seed=33), randn(channels, seed=34)
    want = {b: plain.silu(plain.causal_conv(u[b], weight, bias)) for b in lengths}
    extra = 11  # floats behind the kept inputs, which the kernel must leave alone
    state = torch.zeros(4, (taps - 1) * channels + extra, device=DEV)
    state[:, (taps - 1) * channels:] = 5.0
    done = {b: 0 for b in lengths}
    got = {b: [] for b in lengths}
    steps = [[(0, 1), (1, 2)], [(0, 2), (2, 1)], [(0, 1), (1, 7)], [(0, 5)], [(0, 3)],
             [(0, 11)]]
    for step in steps:
        rows, request_of_row, row_start, slot_of = [], [], [0], []
        for index, (b, n) in enumerate(step):
            rows.append(u[b][done[b]:done[b] + n])
            request_of_row += [index] * n
            row_start.append(row_start[-1] + n)
            slot_of.append(slots[b])
        x = torch.cat(rows).float().to(DEV)
        out = torch.zeros_like(x)
        ops.causal_conv_silu(
            x, weight.float().to(DEV), bias.float().to(DEV), state, out,
            request_of_row=torch.tensor(request_of_row, dtype=torch.int32, device=DEV),
            row_start=torch.tensor(row_start, dtype=torch.int32, device=DEV),
            state_slot=torch.tensor(slot_of, dtype=torch.int32, device=DEV),
            rows=x.shape[0], requests=len(step))
        for index, (b, n) in enumerate(step):
            got[b].append(out[row_start[index]:row_start[index + 1]].cpu())
            done[b] += n
    assert done == lengths
    for b in lengths:
        close(torch.cat(got[b]), want[b], 3e-6, f"request {b}")
    kept = (taps - 1) * channels
    assert float(state[1, :kept].abs().max()) == 0.0 if kept else True  # a slot nobody used
    assert torch.all(state[:, kept:] == 5.0)


# ---- the two recurrences ----------------------------------------------------------------------
def _cuts(total: int, sizes: tuple[int, ...]) -> list[tuple[int, int]]:
    out, at, turn = [], 0, 0
    while at < total:
        size = min(sizes[turn % len(sizes)], total - at)
        out.append((at, at + size))
        at += size
        turn += 1
    return out


@pytest.mark.parametrize("heads, groups, state_size, columns", [
    (2, 1, 4, 5), (4, 2, 16, 16), (3, 3, 40, 24), (2, 2, 130, 33), (1, 1, 300, 9)])
def test_the_state_space_recurrence_whole_and_in_portions(heads, groups, state_size, columns):
    total, inner = 70, heads * columns
    xbc = randn(total, inner + 2 * groups * state_size, seed=40, scale=0.7)
    dt_raw = randn(total, heads, seed=41)
    dt_bias, a_log, skip = randn(heads, seed=42), randn(heads, seed=43, scale=0.5), \
        randn(heads, seed=44)
    dt = torch.nn.functional.softplus(dt_raw + dt_bias)
    decay = torch.exp(-torch.exp(a_log) * dt)
    want = torch.zeros(total, heads, columns, dtype=torch.float64)
    x = xbc[:, :inner].reshape(total, heads, columns)
    B = xbc[:, inner:inner + groups * state_size].reshape(total, groups, state_size)
    C = xbc[:, inner + groups * state_size:].reshape(total, groups, state_size)
    for h in range(heads):
        g = h // (heads // groups)
        S = torch.zeros(state_size, columns, dtype=torch.float64)
        for t in range(total):
            S = decay[t, h] * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            want[t, h] = S.T @ C[t, g] + skip[h] * x[t, h]
    floats = heads * state_size * columns
    for sizes in ((total,), (1,), (2, 33, 1, 5), (32, 3)):
        state = torch.zeros(3, floats + 7, device=DEV)  # slot 1 is used; 7 floats ahead
        y = torch.zeros(total, inner, device=DEV)
        for lo, hi in _cuts(total, sizes):
            ops.mamba2_scan(
                xbc[lo:hi].float().to(DEV), dt_raw[lo:hi].float().to(DEV),
                dt_bias.float().to(DEV), a_log.float().to(DEV), skip.float().to(DEV),
                state[:, 7:], y[lo:hi],
                row_start=torch.tensor([0, hi - lo], dtype=torch.int32, device=DEV),
                state_slot=torch.tensor([1], dtype=torch.int32, device=DEV), requests=1,
                heads=heads, groups=groups, state_size=state_size, columns=columns)
        close(y.reshape(total, heads, columns), want, 1e-5, f"portions {sizes}")
        assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0
        assert float(state[1, :7].abs().max()) == 0.0


@pytest.mark.parametrize("heads, dim, columns, cap", [(1, 4, 3, 5.0), (3, 16, 20, 15.0),
                                                      (2, 72, 48, 8.0), (2, 200, 17, 30.0), (1, 420, 7, 9.0)])
def test_the_matrix_memory_whole_and_in_portions(heads, dim, columns, cap):
    total = 60
    qk, inner = heads * dim, heads * columns
    proj = randn(total, 2 * qk + 2 * inner + 2 * heads, seed=50)
    proj[:, -2 * heads:] *= 6.0  # gates far into the cap on both sides
    bias = randn(2 * heads, seed=51)
    q = proj[:, :qk].reshape(total, heads, dim) * dim ** -0.5
    k = proj[:, qk:2 * qk].reshape(total, heads, dim)
    v = proj[:, 2 * qk:2 * qk + inner].reshape(total, heads, columns)
    i_gate = cap * torch.tanh((proj[:, -2 * heads:-heads] + bias[:heads]) / cap)
    f_gate = torch.nn.functional.logsigmoid(
        cap * torch.tanh((proj[:, -heads:] + bias[heads:]) / cap))
    want = torch.zeros(total, heads, columns, dtype=torch.float64)
    for h in range(heads):
        S = torch.zeros(dim, columns, dtype=torch.float64)
        n = torch.zeros(dim, dtype=torch.float64)
        m = torch.zeros((), dtype=torch.float64)
        for t in range(total):
            m_new = torch.maximum(f_gate[t, h] + m, i_gate[t, h])
            keep, take = torch.exp(f_gate[t, h] + m - m_new), torch.exp(i_gate[t, h] - m_new)
            S = keep * S + take * torch.outer(k[t, h], v[t, h])
            n = keep * n + take * k[t, h]
            m = m_new
            want[t, h] = S.T @ q[t, h] / (torch.maximum((n @ q[t, h]).abs(), torch.exp(-m))
                                          + 1e-6)
    floats = ops.scan_state_floats("mlstm", heads=heads, inner=dim, columns=columns)
    for sizes in ((total,), (1,), (2, 31, 1, 7), (32, 5)):
        state = torch.zeros(2, floats, device=DEV)
        out = torch.zeros(total, inner, device=DEV)
        for lo, hi in _cuts(total, sizes):
            ops.mlstm_scan(
                proj[lo:hi].float().to(DEV), bias.float().to(DEV), state, out[lo:hi],
                row_start=torch.tensor([0, hi - lo], dtype=torch.int32, device=DEV),
                state_slot=torch.tensor([1], dtype=torch.int32, device=DEV), requests=1,
                heads=heads, dim=dim, columns=columns, k_offset=qk, v_offset=2 * qk,
                i_offset=2 * qk + 2 * inner, f_offset=2 * qk + 2 * inner + heads, cap=cap)
        close(out.reshape(total, heads, columns), want, 2e-5, f"portions {sizes}")
        assert float(state[0].abs().max()) == 0.0
