"""The kernels Rizitar added, each against the plain formulas: the element-wise units, routing
over all experts, ungated experts, the delta-rule scan, and the pooled window attention
(prepare, block means, the generic kernel, the kernel of shares, the flash kernel) over
scrambled pages with NaN in every slot that was never written."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_rizitar as plain
from ayaka_b200.parts.pooled_attention import blended_frequencies

pytestmark = pytest.mark.gpu

DEVICE = "cuda"


def _ops():
    from ayaka_b200.kernels import ops
    return ops


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_unary_units(out_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(37, 53, generator=g) * 3).to(DEVICE)
    bias = torch.randn(53, generator=g).to(DEVICE)
    numbers = torch.tensor([0.7, -1.3], device=DEVICE)
    out = torch.empty(40, 53, dtype=out_dtype, device=DEVICE)
    ops.unary_rows(x, out, activation="xielu", rows=37, bias=bias, numbers=numbers)
    want = plain.xielu((x + bias).double().cpu().numpy(), 0.7, -1.3)
    tol = 1e-6 if out_dtype == torch.float32 else 8e-3
    assert np.allclose(out[:37].double().cpu().numpy(), want, rtol=tol, atol=tol)
    ops.unary_rows(x[:, 3:20], out[:, :17], activation="tanh", rows=37)
    assert np.allclose(out[:37, :17].double().cpu().numpy(),
                       np.tanh(x[:, 3:20].double().cpu().numpy()), rtol=tol, atol=tol)


def test_routing_by_the_softmax_over_all_experts():
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    logits = (torch.randn(19, 11, generator=g) * 2).to(DEVICE)
    logits[3, 4] = logits[3, 9] = logits[3].max() + 1  # a tie: the smaller index first
    for top in (1, 3, 11):
        chosen = torch.empty(19 * top, dtype=torch.int32, device=DEVICE)
        share = torch.empty(19 * top, dtype=torch.float32, device=DEVICE)
        ops.moe_route(logits, chosen, share, top=top, rows=19, over_all=True)
        scores = torch.softmax(logits.double(), dim=1).cpu()
        for row in range(19):
            order = sorted(range(11), key=lambda e: (-float(scores[row, e]), e))[:top]
            assert chosen[row * top:(row + 1) * top].tolist() == order
            assert torch.allclose(share[row * top:(row + 1) * top].cpu().double(),
                                  scores[row, order], rtol=1e-5)
    assert chosen.view(19, 11)[3, :2].tolist() == [4, 9]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_without_a_gate(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    rows, width, ff, experts, top = 45, 48, 24, 5, 2
    hidden = torch.randn(rows, width, generator=g).to(DEVICE, dtype)
    w_in = (torch.randn(experts * ff, width, generator=g) / 7).to(DEVICE, dtype)
    w_out = (torch.randn(experts * width, ff, generator=g) / 5).to(DEVICE, dtype)
    chosen = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)])
    chosen = chosen.to(torch.int32).view(-1).to(DEVICE)
    places, tiles = ops.moe_scratch(rows, experts, top)
    sorted_pairs = torch.empty(places, dtype=torch.int32, device=DEVICE)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=DEVICE)
    inner = torch.empty(places, ff, dtype=dtype, device=DEVICE)
    pair_out = torch.full((rows * top, width), float("nan"), device=DEVICE)
    ops.moe_experts(hidden, w_in, w_out, chosen, pair_out, experts=experts, top=top,
                    limit=float("inf"), alpha=1.0, shift=0.0, sorted_pairs=sorted_pairs,
                    tile_expert=tile_expert, inner=inner, rows=rows, single=True)
    h, wi, wo = hidden.double().cpu(), w_in.double().cpu(), w_out.double().cpu()
    for pair in range(rows * top):
        e = int(chosen[pair])
        y = torch.relu(wi[e * ff:(e + 1) * ff] @ h[pair // top]) ** 2
        if dtype == torch.bfloat16:
            y = y.to(torch.bfloat16).double()
        want = wo[e * width:(e + 1) * width] @ y
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(pair_out[pair].double().cpu(), want, rtol=tol,
                              atol=tol * float(want.abs().max())), pair


def _delta_reference(r, k, v, z, y, bias, rate, state):
    """One request, one head: rows in order from ``state`` ``[N, P]`` (float64)."""
    out = []
    for t in range(r.shape[0]):
        w = np.exp(-rate / (1.0 + np.exp(-z[t])))
        a = 1.0 / (1.0 + np.exp(-(y[t] + bias)))
        u = k[t] / math.sqrt(float(k[t] @ k[t]) + 1e-6)
        state[:] = w[:, None] * state - np.outer(a * u, u @ state) + np.outer(k[t], v[t])
        out.append(state.T @ r[t])
    return np.array(out)


@pytest.mark.parametrize("dim,columns", [(5, 5), (12, 20), (40, 16), (64, 64), (100, 33),
                                         (130, 48)])
def test_the_delta_rule_scan(dim, columns):
    """Requests of 1, 3, 70 and 0 + 9 rows in scrambled state slots, run in two steps so that
    the state is carried; key channels and columns that are no multiples of anything."""
    ops = _ops()
    g = torch.Generator().manual_seed(dim)
    heads, rate = 3, 0.61
    qk, inner = heads * dim, heads * columns
    ld = 3 * qk + inner + 7
    k_at, a_at, v_at = qk, 2 * qk, 3 * qk
    slots = [5, 2, 0, 3]
    state = torch.full((6, heads * dim * columns), float("nan"), device=DEVICE)
    state[slots] = 0.0
    bias = (torch.randn(qk, generator=g) * 0.5).to(DEVICE)
    want_state = {b: np.zeros((heads, dim, columns)) for b in range(4)}
    for rows_of in ((1, 3, 70, 9), (2, 1, 37, 1)):
        rows = sum(rows_of)
        proj = torch.randn(rows, ld, generator=g).to(DEVICE)
        decay = (torch.randn(rows, qk, generator=g) * 2).to(DEVICE)
        out = torch.full((rows, inner), float("nan"), device=DEVICE)
        starts = np.concatenate([[0], np.cumsum(rows_of)]).astype(np.int32)
        ops.delta_scan(proj, decay, bias, state, out,
                       row_start=torch.tensor(starts, device=DEVICE),
                       state_slot=torch.tensor(slots, dtype=torch.int32, device=DEVICE),
                       requests=4, heads=heads, dim=dim, columns=columns, k_offset=k_at,
                       v_offset=v_at, a_offset=a_at, decay_rate=rate)
        p, z, b_ = proj.double().cpu().numpy(), decay.double().cpu().numpy(), \
            bias.double().cpu().numpy()
        for b in range(4):
            lo, hi = starts[b], starts[b + 1]
            for h in range(heads):
                want = _delta_reference(
                    p[lo:hi, h * dim:(h + 1) * dim], p[lo:hi, k_at + h * dim:k_at + (h + 1) * dim],
                    p[lo:hi, v_at + h * columns:v_at + (h + 1) * columns],
                    z[lo:hi, h * dim:(h + 1) * dim], p[lo:hi, a_at + h * dim:a_at + (h + 1) * dim],
                    b_[h * dim:(h + 1) * dim], rate, want_state[b][h])
                got = out[lo:hi, h * columns:(h + 1) * columns].double().cpu().numpy()
                assert np.allclose(got, want, rtol=2e-4, atol=2e-4 * np.abs(want).max()), (b, h)
    for b, slot in enumerate(slots):
        got = state[slot].view(heads, columns, dim).transpose(1, 2).double().cpu().numpy()
        assert np.allclose(got, want_state[b], rtol=2e-4, atol=2e-4 * np.abs(want_state[b]).max())
    assert torch.isnan(state[1]).all() and torch.isnan(state[4]).all()  # others' slots untouched


def _attention_case(dtype, heads, kv_heads, dim, window, pool, rot, page, lengths, seed,
                    loud=False):
    """Sequences whose rows are pushed through prepare and the block means in portions, into
    scrambled pages; returns what the attention kernels need and the plain answer."""
    ops = _ops()
    g = torch.Generator().manual_seed(seed)
    q_width, k_width = heads * dim, kv_heads * dim
    scale = 1.7 / math.sqrt(dim)
    freq, gain = blended_frequencies(rot, 300.0, factor=4.0, original=24, fast=6.0, slow=1.0) \
        if rot else ([], 1.0)
    q_w = (1 + 0.2 * torch.randn(dim, generator=g)).to(DEVICE)
    k_w = (1 + 0.2 * torch.randn(dim, generator=g)).to(DEVICE)
    sink = torch.randn(heads, generator=g).to(DEVICE)
    pages_each = [-(-n // page) for n in lengths]
    num_pages = sum(pages_each) + 3
    order = (torch.randperm(num_pages - 1, generator=g) + 1).tolist()  # page 0: none
    table = torch.zeros(len(lengths), max(pages_each), dtype=torch.int32)
    for b, count in enumerate(pages_each):
        for i in range(count):
            table[b, i] = order.pop()
    slots = ops.pool_slots(page, pool) if pool and window else 0
    k_pages = torch.full((num_pages, kv_heads, page, dim), float("nan"), dtype=dtype,
                         device=DEVICE)
    v_pages = torch.full_like(k_pages, float("nan"))
    k_pool = torch.full((num_pages, kv_heads, max(slots, 1), dim), float("nan"), dtype=dtype,
                        device=DEVICE) if slots else None
    v_pool = None if k_pool is None else torch.full_like(k_pool, float("nan"))
    table_d = table.to(DEVICE)
    projections, answers = [], []
    for b, n in enumerate(lengths):
        proj = torch.randn(n, q_width + k_width, generator=g)
        if loud:  # the window's oldest key for the last query, and the block just seen
            proj[max(0, n - window), q_width:] *= 6
            proj[max(0, (max(0, n - window) // pool - 1) * pool), q_width:] *= 6
        projections.append(proj)
        t = {"q": np.eye(q_width, q_width + k_width),
             "k": np.eye(k_width, q_width + k_width, k=q_width),
             "q.norm": q_w.double().cpu().numpy(), "k.norm": k_w.double().cpu().numpy(),
             "sink": sink.double().cpu().numpy(), "o": np.eye(q_width)}
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                 "mask": {"size": window, "pool": pool}}
        if rot:
            mixer["rot"] = {"dims": rot, "base": 300.0, "scaling": {
                "factor": 4.0, "original": 24, "fast": 6.0, "slow": 1.0}}
        answers.append(plain.attention(proj.double().numpy(), t, "", mixer, 1e-5))
        # prepare and block means in portions of 7, 1, 30, ...
        at, turn = 0, 0
        while at < n:
            size = min((7, 1, 30, 2, 64)[turn % 5], n - at)
            turn += 1
            positions = torch.arange(at, at + size, dtype=torch.int32, device=DEVICE)
            pos = positions.cpu()
            mapping = (table[b][pos // page] * page + pos % page).to(torch.int32).to(DEVICE)
            q_scratch = torch.empty(size, q_width, dtype=dtype, device=DEVICE)
            ops.pooled_prepare(
                proj[at:at + size].to(DEVICE), k_offset=q_width, q_weight=q_w, k_weight=k_w,
                eps=1e-5, positions=positions,
                freq=torch.tensor(freq, dtype=torch.float64, device=DEVICE) if rot else None,
                rot_dims=rot, rot_gain=gain, slot_mapping=mapping, k_pages=k_pages,
                v_pages=v_pages, q=q_scratch, heads=heads, kv_heads=kv_heads, dim=dim, rows=size)
            if slots:
                ops.pooled_blocks(k_pages, v_pages, k_pool, v_pool, table_d[b:b + 1],
                                  torch.zeros(size, dtype=torch.int32, device=DEVICE), positions,
                                  torch.tensor([0, size], dtype=torch.int32, device=DEVICE),
                                  pool=pool, rows=size, requests=1)
            at += size
    return dict(ops=ops, projections=projections, answers=answers, table=table_d,
                k_pages=k_pages, v_pages=v_pages, k_pool=k_pool, v_pool=v_pool, sink=sink,
                q_w=q_w, k_w=k_w, freq=freq, gain=gain, scale=scale, q_width=q_width)


def _queries(case, dtype, rows, heads, kv_heads, dim, rot):
    """The queries of the listed (request, position) rows through prepare (nothing stored)."""
    ops = case["ops"]
    proj = torch.stack([case["projections"][b][p] for b, p in rows]).to(DEVICE)
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEVICE)
    q = torch.empty(len(rows), case["q_width"], dtype=dtype, device=DEVICE)
    ops.pooled_prepare(
        proj, k_offset=case["q_width"], q_weight=case["q_w"], k_weight=case["k_w"], eps=1e-5,
        positions=positions,
        freq=torch.tensor(case["freq"], dtype=torch.float64, device=DEVICE) if rot else None,
        rot_dims=rot, rot_gain=case["gain"], slot_mapping=None, k_pages=None, v_pages=None, q=q,
        heads=heads, kv_heads=kv_heads, dim=dim, rows=len(rows))
    return q, positions


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,window,pool,rot,page", [
    (4, 2, 16, 9, 4, 8, 16),      # blocks inside pages
    (3, 1, 24, 21, 5, 24, 8),     # blocks that straddle pages
    (2, 2, 8, 1, 1, 0, 16),       # a window of one, blocks of one, no rotation
    (2, 1, 40, 30, 37, 20, 16),   # a block longer than the window and the page
    (2, 2, 12, 0, 4, 4, 16),      # no window: nothing pooled
])
def test_single_rows_over_scrambled_pages(dtype, heads, kv_heads, dim, window, pool, rot, page):
    lengths = (150, 1, 47, 96)
    case = _attention_case(dtype, heads, kv_heads, dim, window, pool, rot, page, lengths, 5,
                           loud=bool(window and pool))
    ops = case["ops"]
    edges = sorted({0, 1, window - 1, window, window + pool - 1, window + pool,
                    window + 2 * pool - 1, 95, 149} & set(range(150))) if window else [0, 7, 149]
    rows = [(0, p) for p in edges] + [(1, 0), (2, 46), (3, 95), (3, 40)]
    q, positions = _queries(case, dtype, rows, heads, kv_heads, dim, rot)
    request_of_row = torch.tensor([b for b, _ in rows], dtype=torch.int32, device=DEVICE)
    want = torch.tensor(np.stack([case["answers"][b][p] for b, p in rows]))
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for shares in (0, 1, 3, 16):
        if shares and dim % (4 if dtype == torch.float32 else 8):
            continue
        out = torch.full((len(rows), case["q_width"]), float("nan"), dtype=dtype, device=DEVICE)
        partial = torch.empty(len(rows) * heads * max(shares, 1) * (dim + 2), device=DEVICE)
        assert ops.pooled_attention(
            q, case["k_pages"], case["v_pages"], case["k_pool"], case["v_pool"], case["table"],
            request_of_row, positions, out, heads=heads, scale=case["scale"], window=window,
            pool=pool, sink=case["sink"], rows=len(rows), shares=shares, partial=partial)
        got = out.double().cpu()
        assert torch.isfinite(got).all(), shares
        assert float((got - want).abs().max()) <= tol * float(want.abs().max()), shares


@pytest.mark.parametrize("heads,kv_heads,dim,window,pool,rot,page", [
    (4, 2, 32, 40, 3, 16, 16),   # more than a tile of pooled rows behind the last rows
    (2, 1, 64, 64, 12, 64, 16),  # the window ends on a tile's edge
    (2, 2, 16, 5, 7, 8, 8),
])
def test_portions_on_the_flash_kernel(heads, kv_heads, dim, window, pool, rot, page):
    dtype = torch.bfloat16
    lengths = (330, 70, 129)
    case = _attention_case(dtype, heads, kv_heads, dim, window, pool, rot, page, lengths, 9,
                           loud=True)
    ops = case["ops"]
    # the last 200, 70 and 65 rows of the three requests, as one step's portions
    counts = (200, 70, 65)
    rows = [(b, p) for b, n in enumerate(lengths) for p in range(n - counts[b], n)]
    q, _ = _queries(case, dtype, rows, heads, kv_heads, dim, rot)
    starts = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    out = torch.full((len(rows), case["q_width"]), float("nan"), dtype=dtype, device=DEVICE)
    ops.attention_prefill(
        q, case["k_pages"], case["v_pages"], case["table"],
        torch.tensor(starts, device=DEVICE),
        torch.tensor(lengths, dtype=torch.int32, device=DEVICE), out, num_heads=heads,
        scale=case["scale"], host_rows=list(counts), window=window, pool=pool,
        k_pool=case["k_pool"], v_pool=case["v_pool"], sink=case["sink"])
    want = torch.tensor(np.stack([case["answers"][b][p] for b, p in rows]))
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) <= 3e-2 * float(want.abs().max())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [50, 1024, 5000])
def test_the_norm_behind_a_sublayer_applies_the_next_one_too(width, out_dtype):
    """``norm_add`` with the following norm: the stream, its rounding and the next sublayer's
    input from one launch (rows kept in registers, and the wide rows that are not)."""
    ops = _ops()
    g = torch.Generator().manual_seed(width)
    rows = 9
    x = (torch.randn(rows, width, generator=g) * 3).to(DEVICE)
    dst = torch.randn(rows + 2, width, generator=g).to(DEVICE)
    w = (1 + 0.3 * torch.randn(width, generator=g)).to(DEVICE)
    w2 = (1 + 0.3 * torch.randn(width, generator=g)).to(DEVICE)
    before = dst.clone()
    copy = torch.full((rows, width), float("nan"), dtype=out_dtype, device=DEVICE)
    nxt = torch.full((rows, width), float("nan"), dtype=out_dtype, device=DEVICE)
    ops.norm_add(x, w, 1e-5, dst, factor=0.7, weight_offset=0.25, copy=copy, rows=rows,
                 next_weight=w2, next_eps=1e-3, next_offset=0.5, next_out=nxt)
    want = before[:rows].double().cpu().numpy() + 0.7 * plain.rms(
        x.double().cpu().numpy(), 0.25 + w.double().cpu().numpy(), 1e-5)
    want_next = plain.rms(want, 0.5 + w2.double().cpu().numpy(), 1e-3)
    tol = 1e-5 if out_dtype == torch.float32 else 8e-3
    assert np.allclose(dst[:rows].double().cpu().numpy(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(dst[rows:], before[rows:])
    assert np.allclose(copy.double().cpu().numpy(), want, rtol=tol, atol=tol)
    assert np.allclose(nxt.double().cpu().numpy(), want_next, rtol=tol, atol=tol)
