"""The kernels Semadra brought, each alone against a plain float64 formula, at sizes of their
own, with the inputs arranged so that a fault shows: a window's edge, the end of the kept
stretch, a page's border, shuffled pages, a far loud key."""

from __future__ import annotations

import math

import pytest
import torch

import plain_semadra as plain
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


# ---- the stream: casts, output norms, gated units ---------------------------------------------
@pytest.mark.parametrize("width", [24, 130, 1024])
@pytest.mark.parametrize("copy_dtype", [None, torch.float32, torch.bfloat16])
def test_norm_add_with_a_factor_an_offset_and_a_copy(width, copy_dtype):
    rows, eps, factor = 7, 3e-4, 0.35
    x, w = randn(rows + 2, width, seed=1, scale=4.0), randn(width, seed=2, scale=0.3)
    dst = randn(rows + 2, width, seed=3)
    got = dst.float().to(DEV)
    copy = None if copy_dtype is None else torch.zeros(rows + 2, width, dtype=copy_dtype,
                                                       device=DEV)
    ops.norm_add(x.float().to(DEV), w.float().to(DEV), eps, got, factor=factor,
                 weight_offset=1.0, copy=copy, rows=rows)
    want = dst.float().double().clone()
    want[:rows] += factor * plain.rms(x.float().double()[:rows], eps) * (1 + w.float().double())
    close(got, want, 2e-6, "sum")
    assert torch.equal(got[rows:].cpu(), dst.float()[rows:])  # rows beyond the count stay
    if copy is not None:
        assert torch.equal(copy[:rows], got[:rows].to(copy_dtype))  # rounded once, from the sum
        assert float(copy[rows:].abs().max()) == 0.0
    plain_weight = dst.float().to(DEV)
    ops.norm_add(x.float().to(DEV), w.float().to(DEV), eps, plain_weight, rows=rows)
    close(plain_weight[:rows], dst.float().double()[:rows]
          + plain.rms(x.float().double()[:rows], eps) * w.float().double(), 2e-6, "plain weight")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gated_unit_with_another_row_and_with_a_table(out_dtype, activation):
    rows, width, vocab = 11, 20, 9
    tol = 3e-6 if out_dtype == torch.float32 else 5e-3
    gate, other = randn(rows, width, seed=4, scale=3.0), randn(rows, width, seed=5)
    act = plain.silu if activation == "silu" else plain.gelu_tanh
    out = torch.zeros(rows, width, dtype=out_dtype, device=DEV)
    ops.gated_unit(gate.float().to(DEV), out, activation=activation, rows=rows,
                   other=other.float().to(DEV))
    close(out, act(gate.float().double()) * other.float().double(), tol, "two rows")
    # a table wider than the unit: its columns 6 .. 26 of the row's own token
    table = randn(vocab, width + 13, seed=6).to(out_dtype)
    index = torch.tensor([8, 0, 3, 3, 7, 1, 2, 8, 4, 5, 6], dtype=torch.int32)
    out.zero_()
    ops.gated_unit(gate.float().to(DEV), out, activation=activation, rows=rows,
                   table=table.to(DEV), index=index.to(DEV), column=6)
    want = act(gate.float().double()) * table.double()[index.long(), 6:6 + width]
    close(out, want, tol, "table")


def test_cast_rows():
    x = randn(5, 70, seed=7, scale=100.0).float()
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.zeros(6, 70, dtype=dtype, device=DEV)
        ops.cast_rows(x.to(DEV), out, rows=5)
        assert torch.equal(out[:5].cpu(), x.to(dtype)) and float(out[5].abs().max()) == 0.0


# ---- routing by scores among the best groups --------------------------------------------------
@pytest.mark.parametrize("experts, top, groups, keep, factor, renormalise", [
    (12, 3, 4, 3, 2.0, False), (6, 2, 3, 2, 1.5, False), (5, 3, 5, 4, 2.5, False),
    (8, 2, 2, 1, 1.0, True), (4, 1, 1, 1, 0.7, False), (64, 8, 8, 4, 2.5, True),
    (24, 4, 6, 2, 0.5, False), (3, 3, 1, 1, 1.0, False), (256, 8, 8, 4, 2.5, False)])
def test_routing_by_scores(experts, top, groups, keep, factor, renormalise):
    rows = 97
    logits = randn(rows, experts, seed=experts + top, scale=2.0).float()
    chosen = torch.zeros(rows * top, dtype=torch.int32, device=DEV)
    share = torch.zeros(rows * top, dtype=torch.float32, device=DEV)
    ops.moe_route_scored(logits.to(DEV), chosen, share, top=top, groups=groups, keep=keep,
                         factor=factor, renormalise=renormalise, rows=rows)
    scores = torch.sigmoid(logits.double())
    want = plain.expert_choice(scores, top, groups, keep)
    got = chosen.cpu().reshape(rows, top).long()
    safe = plain.choice_margin(scores, top, groups, keep) > 1e-6
    assert int(safe.sum()) > rows * 0.9
    assert torch.equal(got[safe].sort(dim=1).values, want[safe].sort(dim=1).values)
    weights = scores.gather(1, got)
    if renormalise:
        weights = weights / weights.sum(dim=1, keepdim=True)
    close(share.cpu().reshape(rows, top)[safe], (factor * weights)[safe], 3e-6, "weights")


def test_routing_by_scores_by_hand():
    """Groups of two: the second largest score of all sits in a group that is not kept."""
    scores = torch.tensor([[0.9, 0.1, 0.6, 0.5, 0.8, 0.05]], dtype=torch.float64)
    logits = torch.log(scores / (1 - scores)).float()
    chosen = torch.zeros(2, dtype=torch.int32, device=DEV)
    share = torch.zeros(2, dtype=torch.float32, device=DEV)
    ops.moe_route_scored(logits.to(DEV), chosen, share, top=2, groups=3, keep=2, factor=2.0,
                         rows=1)
    assert chosen.cpu().tolist() == [0, 2]
    close(share, torch.tensor([1.8, 1.2], dtype=torch.float64), 1e-6)


# ---- attention with kept first tokens, grouped heads, a value size of its own, a gate ---------
def _paged(rows_of_request: list[torch.Tensor], page: int, dtype, order: list[int], total: int):
    """Scatter each request's rows ``[T, G, D]`` over pages ``[page, G, slot, D]`` handed out
    in the given order (the same order for keys and values); unwritten slots hold NaN."""
    groups, width = rows_of_request[0].shape[1:]
    need = [-(-t.shape[0] // page) for t in rows_of_request]
    pages = torch.full((total, groups, page, width), float("nan"), dtype=torch.float64)
    table = torch.zeros(len(need), max(need), dtype=torch.int32)
    at = 0
    for b, rows in enumerate(rows_of_request):
        for index in range(need[b]):
            page_id = order[at]
            at += 1
            table[b, index] = page_id
            piece = rows[index * page:(index + 1) * page]
            pages[page_id, :, :piece.shape[0]] = piece.transpose(0, 1)
    return pages.to(dtype).to(DEV), table.to(DEV)


CASES = [
    # heads, kv heads, dim, vdim, window, keep_first, page
    (4, 2, 16, 8, 9, 13, 8),
    (3, 1, 8, 20, 1, 0, 16),
    (2, 2, 12, 6, 0, 0, 16),
    (6, 3, 32, 16, 40, 24, 16),
    (2, 1, 64, 64, 70, 5, 32),
    (5, 5, 24, 40, 33, 1, 16),
    (8, 2, 128, 128, 100, 17, 16),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("rows_kind, shares", [("ends", 0), ("portions", 0), ("ends", 1),
                                               ("ends", 3), ("portions", 16)])
def test_gated_attention_sees_its_window_and_the_kept_tokens_and_not_a_key_more(
        dtype, case, rows_kind, shares):
    """Three keys are made to stand out for every query asked: the last kept one, the oldest
    one in its window, and, louder than both, the one just before the window that is not
    kept. The first two share nearly all the weight, the third gets none. ``ends``: single
    rows at the ends of sequences (a decode step); ``portions``: the last rows of every
    sequence together (prompt portions, beside single rows). ``shares`` > 0: the kernel of
    single rows, which cuts a row's visible keys into that many shares (more shares than
    some rows have keys), with a row of padding at the end."""
    heads, groups, dim, vdim, window, keep, page = case
    if shares and vdim % (4 if dtype == torch.float32 else 8):
        pytest.skip("value rows that are no whole 16-byte pieces go to the other kernel")
    lengths = [1, 2, page, page + 1, 3 * page - 1, 150, 333]
    per = heads // groups
    direction = randn(dim, seed=9)
    direction = direction / direction.norm()
    keys = [randn(t, groups, dim, seed=20 + i, scale=0.3) for i, t in enumerate(lengths)]
    values = [randn(t, groups, vdim, seed=40 + i) for i, t in enumerate(lengths)]
    queries, request_of_row, positions = [], [], []
    for b, t in enumerate(lengths):
        first = t - 1 if rows_kind == "ends" else max(0, t - (1 if b % 2 else 70))
        for p in range(first, t):
            queries.append(randn(heads, dim, seed=1000 * b + p, scale=0.5) + 3.0 * direction)
            request_of_row.append(b)
            positions.append(p)
        p = t - 1  # the loud keys are placed for the last row of each request
        oldest = max(0, p - window + 1) if window else 0
        keys[b][oldest] += 5.0 * direction
        if oldest > keep:
            keys[b][oldest - 1] += 10.0 * direction
        if keep and oldest > keep:
            keys[b][keep - 1] += 5.0 * direction
    keys = [k.to(dtype).double() for k in keys]
    values = [v.to(dtype).double() for v in values]
    q = torch.stack(queries).to(dtype)
    need = sum(-(-t // page) for t in lengths)
    order = (torch.randperm(need, generator=gen(3)) + 1).tolist()
    k_pages, table = _paged(keys, page, dtype, order, need + 1)
    v_pages, _ = _paged(values, page, dtype, order, need + 1)
    n, scale = len(positions), 0.8
    gate = randn(n, heads * vdim, seed=77, scale=2.0).float()
    out = torch.full((n + 1, heads * vdim), 7.0, dtype=dtype, device=DEV)
    if shares:
        partial = torch.full(((n + 1) * heads * shares * (vdim + 2),), float("nan"),
                             device=DEV)
        out = torch.full((n + 2, heads * vdim), 7.0, dtype=dtype, device=DEV)
        assert ops.gated_decode(
            torch.cat([q.reshape(n, heads * dim), q.reshape(n, heads * dim)[:1]]).to(DEV),
            k_pages, v_pages, table,
            torch.tensor(request_of_row + [-1], dtype=torch.int32, device=DEV),
            torch.tensor(positions + [0], dtype=torch.int32, device=DEV), out, partial,
            heads=heads, scale=scale, window=window, keep_first=keep,
            gate=torch.cat([gate, gate[:1]]).to(DEV), rows=n + 1, shares=shares)
        assert float(out[n].float().abs().max()) == 0.0  # the row of padding
        assert float((out[n + 1] - 7.0).abs().max()) == 0.0
        out = torch.cat([out[:n], out[n + 1:]])
    else:
        ops.gated_attention(q.reshape(n, heads * dim).to(DEV), k_pages, v_pages, table,
                            torch.tensor(request_of_row, dtype=torch.int32, device=DEV),
                            torch.tensor(positions, dtype=torch.int32, device=DEV), out,
                            heads=heads, scale=scale, window=window, keep_first=keep,
                            gate=gate.to(DEV), rows=n)
    got = out[:n].double().cpu().reshape(n, heads, vdim)
    assert torch.isfinite(got).all() and float((out[n] - 7.0).abs().max()) == 0.0
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for i, (b, p) in enumerate(zip(request_of_row, positions)):
        mask = plain.visible(p + 1, window or p + 1, keep)[p]
        for h in range(heads):
            scores = scale * (keys[b][:p + 1, h // per] @ q[i, h].double())
            weights = torch.softmax(scores.masked_fill(~mask, -math.inf), dim=-1)
            want = (weights @ values[b][:p + 1, h // per]) * \
                torch.sigmoid(gate[i].double().reshape(heads, vdim)[h])
            close(got[i, h], want, tol, f"request {b} position {p} head {h}")


TILED_CASES = [
    # heads, kv heads, dim, vdim, window, keep_first, page
    (6, 3, 32, 16, 40, 24, 16),
    (2, 1, 64, 64, 70, 5, 32),
    (4, 2, 48, 80, 130, 70, 16),   # kept keys beyond one tile of keys
    (2, 2, 16, 32, 64, 64, 8),     # the window and the kept stretch end on a tile's edge
    (3, 1, 128, 16, 0, 9, 16),     # no window: nothing is kept apart
    (2, 1, 32, 32, 5, 200, 16),    # everything is kept
]


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("case", TILED_CASES)
def test_the_tiled_kernel_takes_the_kept_tokens_a_value_size_and_a_gate(case, gated):
    """Prompt portions of several lengths (one row to more than four tiles of rows) on the
    tensor-core kernel. For the last row of every request the last kept key, the oldest key
    of the window and, louder, the key just before the window are made to stand out."""
    heads, groups, dim, vdim, window, keep, page = case
    lengths = [1, 2, 17, 65, 150, 333, 400]
    tails = [1, 2, 17, 3, 150, 70, 270]
    per, dtype = heads // groups, torch.bfloat16
    direction = randn(dim, seed=9)
    direction = direction / direction.norm()
    keys = [randn(t, groups, dim, seed=20 + i, scale=0.3) for i, t in enumerate(lengths)]
    values = [randn(t, groups, vdim, seed=40 + i) for i, t in enumerate(lengths)]
    queries, request_of_row, positions, row_start = [], [], [], [0]
    for b, (t, tail) in enumerate(zip(lengths, tails)):
        for p in range(t - tail, t):
            queries.append(randn(heads, dim, seed=1000 * b + p, scale=0.5) + 3.0 * direction)
            request_of_row.append(b)
            positions.append(p)
        row_start.append(len(positions))
        p = t - 1
        oldest = max(0, p - window + 1) if window else 0
        keys[b][oldest] += 5.0 * direction
        if oldest > keep:
            keys[b][oldest - 1] += 10.0 * direction
        if keep and oldest > keep:
            keys[b][keep - 1] += 5.0 * direction
    keys = [k.to(dtype).double() for k in keys]
    values = [v.to(dtype).double() for v in values]
    q = torch.stack(queries).to(dtype)
    need = sum(-(-t // page) for t in lengths)
    order = (torch.randperm(need, generator=gen(4)) + 1).tolist()
    k_pages, table = _paged(keys, page, dtype, order, need + 1)
    v_pages, _ = _paged(values, page, dtype, order, need + 1)
    n, scale = len(positions), 0.8
    gate = randn(n, heads * vdim, seed=78, scale=2.0).float()
    out = torch.full((n + 1, heads * vdim), 7.0, dtype=dtype, device=DEV)
    ops.attention_prefill(q.reshape(n, heads * dim).to(DEV), k_pages, v_pages, table,
                          torch.tensor(row_start, dtype=torch.int32, device=DEV),
                          torch.tensor(lengths, dtype=torch.int32, device=DEV), out,
                          num_heads=heads, scale=scale, host_rows=tails, window=window,
                          keep_first=keep, gate=gate.to(DEV) if gated else None)
    got = out[:n].double().cpu().reshape(n, heads, vdim)
    assert torch.isfinite(got).all() and float((out[n] - 7.0).abs().max()) == 0.0
    for i, (b, p) in enumerate(zip(request_of_row, positions)):
        if i % 3 and p != lengths[b] - 1 and p % 64 not in (0, 63):
            continue  # every third row, the tiles' edges and the rows with the loud keys
        mask = plain.visible(p + 1, window or p + 1, keep if window else 0)[p]
        for h in range(heads):
            scores = scale * (keys[b][:p + 1, h // per] @ q[i, h].double())
            weights = torch.softmax(scores.masked_fill(~mask, -math.inf), dim=-1)
            want = weights @ values[b][:p + 1, h // per]
            if gated:
                want = want * torch.sigmoid(gate[i].double().reshape(heads, vdim)[h])
            close(got[i, h], want, 1.5e-2, f"request {b} position {p} head {h}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prepare_norms_the_whole_projections_and_stores_where_the_slots_say(dtype):
    heads, groups, dim, vdim, page, rows, eps = 4, 2, 12, 20, 8, 10, 1e-3
    qn, kn, vn = heads * dim, groups * dim, groups * vdim
    k_off, v_off = qn + 3, qn + 3 + kn + 5  # gaps between the pieces
    proj = randn(rows, v_off + vn + 7, seed=11, scale=3.0).float()
    wq, wk = randn(qn, seed=12).float(), randn(kn, seed=13).float()
    slots = torch.tensor([17, 3, 40, 41, 8, 9, 10, 63, 0, 25], dtype=torch.int32)
    k_pages = torch.zeros(8, groups, page, dim, dtype=dtype, device=DEV)
    v_pages = torch.zeros(8, groups, page, vdim, dtype=dtype, device=DEV)
    q = torch.zeros(rows, qn, dtype=dtype, device=DEV)
    ops.gated_attention_prepare(proj.to(DEV), k_offset=k_off, v_offset=v_off,
                                q_weight=wq.to(DEV), k_weight=wk.to(DEV), eps=eps,
                                slot_mapping=slots.to(DEV), k_pages=k_pages, v_pages=v_pages,
                                q=q, heads=heads, kv_heads=groups, dim=dim, vdim=vdim, rows=rows)
    tol = 3e-6 if dtype == torch.float32 else 5e-3
    wide = proj.double()
    close(q, plain.rms(wide[:, :qn], eps) * wq.double(), tol, "queries")
    want_k = (plain.rms(wide[:, k_off:k_off + kn], eps) * wk.double()).reshape(rows, groups, dim)
    want_v = wide[:, v_off:v_off + vn].reshape(rows, groups, vdim)
    for r, slot in enumerate(slots.tolist()):
        close(k_pages[slot // page, :, slot % page], want_k[r], tol, f"key of row {r}")
        close(v_pages[slot // page, :, slot % page], want_v[r], tol, f"value of row {r}")
    assert int((k_pages.float().abs().sum(dim=(1, 3)) > 0).sum()) == rows  # nothing else
    # without weights and pages: queries as projected, nothing stored
    k_pages.zero_()
    ops.gated_attention_prepare(proj.to(DEV), k_offset=k_off, v_offset=v_off, q_weight=None,
                                k_weight=None, eps=eps, slot_mapping=None, k_pages=None,
                                v_pages=None, q=q, heads=heads, kv_heads=groups, dim=dim,
                                vdim=vdim, rows=rows)
    close(q, wide[:, :qn], tol, "queries as projected")
    assert float(k_pages.float().abs().max()) == 0.0
