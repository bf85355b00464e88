"""The kernels as functions over torch tensors.

Every function writes into tensors the caller allocated and launches on torch's current
CUDA stream. Tensors are on one CUDA device; 2-D tensors may have any row stride but a unit
stride along the last dimension. Nothing here falls back to torch arithmetic: a missing
library or a refused argument raises :class:`~ayaka_b200.errors.BackendError`.
"""

from __future__ import annotations

import contextlib
import math
from collections.abc import Iterator
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ayaka_b200.errors import BackendError
from ayaka_b200.kernels.lib import check, library, raw_stream

__all__ = [
    "ACTIVATIONS",
    "argmax",
    "attention",
    "attention_decode",
    "attention_prefill",
    "cast_rows",
    "causal_conv_silu",
    "decode_splits",
    "delta_scan",
    "embed_rows",
    "gated_attention",
    "gated_attention_prepare",
    "gated_decode",
    "gated_decode_shares",
    "gated_unit",
    "head_linear",
    "kv_store",
    "latent_attention",
    "latent_decode",
    "latent_prepare",
    "launch_count",
    "leaving_out",
    "gla_scan",
    "layer_norm",
    "linear",
    "linear_normed",
    "logits_adjust",
    "logits_scale_cap",
    "mamba2_scan",
    "mlstm_scan",
    "moe_experts",
    "moe_join",
    "moe_max_tiles",
    "moe_route",
    "moe_route_scored",
    "moe_scratch",
    "moe_tile_rows",
    "norm_add",
    "norm_sum",
    "pool_slots",
    "pooled_attention",
    "pooled_blocks",
    "pooled_prepare",
    "rms_norm",
    "rope",
    "rope_frequencies",
    "sample",
    "scale_add",
    "scan_state_floats",
    "set_decode_tensor_cores",
    "set_pdl",
    "sm_count",
    "talking_attention",
    "talking_prepare",
    "timed",
    "unary_rows",
]

ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2}
_TYPE = {torch.float32: 0, torch.bfloat16: 1}

#: Which bfloat16 matrix-product kernel :func:`linear` launches: ``"tcgen05"`` (the tensor
#: cores, the serving path) or ``"simt"`` (the CUDA-core reference); tests switch it.
BF16_GEMM = "tcgen05"


#: Whether parts that can hand a layer half (or a run of layers) to the C++ host code
#: (``csrc/step_host.cu``) do so; tests switch it off to compare the two paths bit by bit.
NATIVE_STEP = True

#: How :class:`~ayaka_b200.parts.pooled_attention.PooledWindowAttention` runs bfloat16 prompt
#: portions: ``"mma"`` (the flash kernel on the tensor cores) or ``"generic"`` (one CTA per
#: row and head on the CUDA cores); tests switch it to compare the two.
POOLED_PREFILL = "mma"

_launches = 0

#: Kernel classes that launch nothing while a measurement runs; empty in normal use. A
#: class is an operation's name, for matrix products with the weight's shape
#: (``"linear:4800x1600"``). ``bench.py`` times a step with and without each class inside
#: the same chain of dependent launches, which is what a kernel costs there; a step with a
#: class left out computes nothing meaningful.
_left_out: frozenset[str] = frozenset()


@contextlib.contextmanager
def leaving_out(*classes: str) -> Iterator[None]:
    """Within the block the named kernel classes are not launched (for measurements only)."""
    global _left_out
    before = _left_out
    _left_out = before | frozenset(classes)
    try:
        yield
    finally:
        _left_out = before


_TIMED = ("embed_rows", "layer_norm", "linear", "linear_kv", "kv_store", "attention",
          "attention_prefill", "attention_decode", "argmax", "sample", "rms_norm", "rope",
          "latent_prepare", "head_linear", "latent_attention", "latent_decode",
          "causal_conv_silu", "mamba2_scan",
          "mlstm_scan", "gla_scan", "talking_prepare", "talking_attention", "norm_sum",
          "moe_route", "moe_experts", "moe_join", "moe_route_scored", "cast_rows", "gated_unit",
          "norm_add", "gated_attention_prepare", "gated_attention", "gated_decode",
          "unary_rows", "delta_scan", "pooled_prepare", "pooled_blocks", "pooled_attention")


@contextlib.contextmanager
def timed() -> Iterator[dict[str, list[tuple[torch.cuda.Event, torch.cuda.Event]]]]:
    """Within the block every launch through this module is bracketed by two CUDA events,
    gathered per kernel class (see ``leaving_out`` for the names); after a synchronisation
    ``start.elapsed_time(stop)`` of each pair is that kernel's own duration. The events keep
    a kernel from starting under its predecessor's tail, so this suits steps of large
    kernels (prompt portions), not decode chains. For measurements only."""
    module = globals()
    originals = {name: module[name] for name in _TIMED}
    record: dict[str, list[tuple[torch.cuda.Event, torch.cuda.Event]]] = {}

    def wrap(name: str, function):  # noqa: ANN001, ANN202
        def wrapped(*args, **kwargs):  # noqa: ANN002, ANN003, ANN202
            klass = name
            if name in ("linear", "linear_kv"):
                klass = f"linear:{args[1].shape[0]}x{args[1].shape[1]}"
            elif name == "gated_decode" or name == "attention_prefill" and (
                    kwargs.get("gate") is not None or kwargs.get("keep_first")):
                klass = "gated_attention"  # that part's single rows and prompt portions
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            result = function(*args, **kwargs)
            stop.record()
            record.setdefault(klass, []).append((start, stop))
            return result
        return wrapped

    for name, function in originals.items():
        module[name] = wrap(name, function)
    try:
        yield record
    finally:
        module.update(originals)


def set_pdl(enabled: bool) -> None:
    """Switch programmatic dependent launch on or off in every library (it is on by default;
    measurements switch it off to see what it buys). Graphs captured earlier keep their edges."""
    from ayaka_b200.kernels import lib

    lib.set_pdl(enabled)


def set_decode_tensor_cores(enabled: bool) -> None:
    """Let decode attention choose its tensor-core kernel where that serves the case (the
    default), or keep every call on the split-KV kernel (tests of that kernel at head sizes
    64 and 128 in bfloat16, and measurements of one kernel against the other)."""
    library("attention_decode").ayk_set_decode_tensor_cores(c_int(1 if enabled else 0))


def launch_count() -> int:
    """Kernels launched through this module since the process started (a graph capture
    counts the kernels it records)."""
    return _launches


def _status_word(device: torch.device) -> torch.Tensor:
    from ayaka_b200.kernels import gemm_tc

    return gemm_tc.status_word(device)


def _stream() -> c_void_p:
    global _launches
    _launches += 1
    return c_void_p(raw_stream())


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())


def _need(op: str, name: str, tensor: torch.Tensor, dtype: torch.dtype | None = None,
          ndim: int | None = None) -> None:
    if not tensor.is_cuda:
        raise BackendError(f"{op}: {name} must be on a CUDA device, it is on {tensor.device}")
    if dtype is not None and tensor.dtype != dtype:
        raise BackendError(f"{op}: {name} must be {dtype}, got {tensor.dtype}")
    if ndim is not None and tensor.ndim != ndim:
        raise BackendError(f"{op}: {name} must have {ndim} dimensions, got {tensor.ndim}")
    if tensor.ndim and tensor.numel() and tensor.stride(-1) != 1:
        raise BackendError(f"{op}: {name} must have a unit stride along its last dimension")


def embed_rows(table: torch.Tensor, index: torch.Tensor, out: torch.Tensor, *,
               add_table: torch.Tensor | None = None, add_index: torch.Tensor | None = None,
               bad_index: torch.Tensor, scale: float = 1.0) -> None:
    """``out[i] = scale * table[index[i]] (+ add_table[add_index[i]])`` as fp32 rows.

    ``bad_index`` is one int32 on the device that the kernel sets to 1 if an id is outside
    its table.
    """
    op = "embed_rows"
    if _left_out and op in _left_out:
        return
    _need(op, "table", table, ndim=2)
    _need(op, "index", index, torch.int32, 1)
    _need(op, "out", out, torch.float32, 2)
    _need(op, "bad_index", bad_index, torch.int32)
    if table.dtype not in _TYPE or not table.is_contiguous():
        raise BackendError(f"{op}: table must be contiguous float32 or bfloat16")
    rows, width = index.shape[0], table.shape[1]
    if out.shape[0] < rows or out.shape[1] != width:
        raise BackendError(f"{op}: out {list(out.shape)} does not hold [{rows}, {width}]")
    if add_table is not None:
        if add_index is None:
            raise BackendError(f"{op}: add_table needs add_index")
        _need(op, "add_table", add_table, table.dtype, 2)
        _need(op, "add_index", add_index, torch.int32, 1)
        if add_table.shape[1] != width or add_index.shape[0] != rows or \
                not add_table.is_contiguous():
            raise BackendError(f"{op}: add_table/add_index do not match the rows")
    name = "ayk_embed_rows_f32" if table.dtype == torch.float32 else "ayk_embed_rows_bf16"
    fn = getattr(library("embed"), name)
    status = fn(_ptr(table), _ptr(index), c_int(table.shape[0]), _ptr(add_table),
                _ptr(add_index), c_int(0 if add_table is None else add_table.shape[0]),
                _ptr(out), c_int(out.stride(0)), c_int(rows), c_int(width), c_float(scale),
                _ptr(bad_index), _stream())
    check(status, op)


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float,
               out: torch.Tensor, *, rows: torch.Tensor | None = None,
               count: int | None = None) -> None:
    """LayerNorm of fp32 rows into ``out`` (float32 or bfloat16).

    With ``rows`` (int32), output row ``i`` normalises ``x[rows[i]]``. ``count`` limits the
    number of output rows (default: all of ``rows`` or of ``x``).
    """
    op = "layer_norm"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "gamma", gamma, torch.float32, 1)
    if beta is not None:
        _need(op, "beta", beta, torch.float32, 1)
    _need(op, "out", out, ndim=2)
    if out.dtype not in _TYPE:
        raise BackendError(f"{op}: out must be float32 or bfloat16, got {out.dtype}")
    width = x.shape[1]
    if gamma.shape[0] != width or (beta is not None and beta.shape[0] != width) or \
            out.shape[1] != width:
        raise BackendError(f"{op}: widths differ")
    if rows is not None:
        _need(op, "rows", rows, torch.int32, 1)
    n = count if count is not None else (rows.shape[0] if rows is not None else x.shape[0])
    if n > out.shape[0] or (rows is None and n > x.shape[0]) or \
            (rows is not None and n > rows.shape[0]):
        raise BackendError(f"{op}: {n} rows do not fit the tensors")
    name = "ayk_layer_norm_f32" if out.dtype == torch.float32 else "ayk_layer_norm_bf16"
    fn = getattr(library("norm"), name)
    status = fn(_ptr(x), c_int(x.stride(0)), _ptr(rows), _ptr(gamma), _ptr(beta),
                c_float(eps), _ptr(out), c_int(out.stride(0)), c_int(n), c_int(width), _stream())
    check(status, op)


def linear(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
           *, activation: str = "none", residual: bool = False, rows: int | None = None,
           kernel: str | None = None) -> None:
    """``out = act(a @ weight.T + bias)``, or ``out += a @ weight.T + bias`` with ``residual``.

    ``a`` is ``[M, K]``, ``weight`` ``[N, K]`` (both float32, or both bfloat16), ``bias``
    float32 ``[N]``. ``out`` is ``[M, N]``: float32 always allowed (and required with
    ``residual``), bfloat16 for bfloat16 inputs. ``rows`` limits M. float32 inputs run on
    the CUDA cores with fp32 FMA (no reduced-precision matrix mode); bfloat16 inputs on the
    tensor cores unless ``kernel="simt"``.
    """
    op = "linear"
    if _left_out and f"linear:{weight.shape[0]}x{weight.shape[1]}" in _left_out:
        return
    _need(op, "a", a, ndim=2)
    _need(op, "weight", weight, a.dtype, 2)
    _need(op, "out", out, ndim=2)
    if a.dtype not in _TYPE or out.dtype not in _TYPE:
        raise BackendError(f"{op}: float32 and bfloat16 only, got {a.dtype} -> {out.dtype}")
    if bias is not None:
        _need(op, "bias", bias, torch.float32, 1)
    m = a.shape[0] if rows is None else rows
    n, k = weight.shape
    if a.shape[1] != k or m > a.shape[0] or m > out.shape[0] or out.shape[1] != n or \
            (bias is not None and bias.shape[0] != n):
        raise BackendError(
            f"{op}: shapes a{list(a.shape)} w{list(weight.shape)} out{list(out.shape)} "
            f"rows={m} do not fit")
    if activation not in ACTIVATIONS:
        raise BackendError(f"{op}: unknown activation {activation!r}")
    if residual and (out.dtype != torch.float32 or activation != "none"):
        raise BackendError(f"{op}: a residual sum is float32 and has no activation")
    if a.dtype == torch.float32 and out.dtype != torch.float32:
        raise BackendError(f"{op}: float32 inputs give float32 output")
    which = kernel or (BF16_GEMM if a.dtype == torch.bfloat16 else "simt")
    if which == "tcgen05" and a.dtype == torch.bfloat16:
        from ayaka_b200.kernels import gemm_tc

        # operands TMA cannot read (a row stride that is no multiple of 8 elements) go to
        # the CUDA-core kernel: slower, same result
        if kernel == "tcgen05" or gemm_tc.usable(a, weight):
            gemm_tc.linear_bf16(a, weight, bias, out, m, ACTIVATIONS[activation], residual)
            return
    fn = library("gemm_simt").ayk_gemm_simt
    status = fn(_ptr(a), c_int(a.stride(0)), _ptr(weight), c_int(weight.stride(0)), _ptr(bias),
                _ptr(out), c_int(out.stride(0)), c_int(m), c_int(n), c_int(k),
                c_int(ACTIVATIONS[activation]), c_int(1 if residual else 0),
                c_int(_TYPE[a.dtype]), c_int(_TYPE[out.dtype]), _stream())
    check(status, op)


def linear_kv(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
              out: torch.Tensor, slot_mapping: torch.Tensor, k_pages: torch.Tensor,
              v_pages: torch.Tensor, *, q_width: int, rows: int | None = None) -> bool:
    """``a @ weight.T + bias`` for a fused query/key/value projection (bfloat16): the query
    columns go to ``out[:, :q_width]``; the key and value columns (keys, then values) go into
    the cache pages at ``slot_mapping``, written by the product's own epilogue, and **not**
    to ``out`` (whose columns from ``q_width`` on keep what they held). Returns False, having
    done nothing, when that cannot be had (float32, few rows, sizes the kernel does not
    take): the caller then runs :func:`linear` and :func:`kv_store`."""
    op = "linear_kv"
    if _left_out and f"linear:{weight.shape[0]}x{weight.shape[1]}" in _left_out:
        return True
    if a.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or BF16_GEMM != "tcgen05":
        return False
    _need(op, "a", a, torch.bfloat16, 2)
    _need(op, "weight", weight, torch.bfloat16, 2)
    _need(op, "out", out, torch.bfloat16, 2)
    _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
    _need(op, "k_pages", k_pages, torch.bfloat16, 4)
    _need(op, "v_pages", v_pages, torch.bfloat16, 4)
    if bias is not None:
        _need(op, "bias", bias, torch.float32, 1)
    m = a.shape[0] if rows is None else rows
    n, k = weight.shape
    _, kv_heads, _, head_dim = k_pages.shape
    if a.shape[1] != k or m > a.shape[0] or m > out.shape[0] or out.shape[1] != n or \
            m > slot_mapping.shape[0] or n != q_width + 2 * kv_heads * head_dim or \
            v_pages.shape != k_pages.shape or (bias is not None and bias.shape[0] != n):
        raise BackendError(f"{op}: shapes do not fit")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous pages only")
    from ayaka_b200.kernels import gemm_tc

    return gemm_tc.linear_bf16_kv(a, weight, bias, out, m, slot_mapping, k_pages, v_pages,
                                  q_width)


def linear_normed(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float,
                  weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, *,
                  scratch: torch.Tensor, count: int, activation: str = "none",
                  row_index: torch.Tensor | None = None) -> None:
    """``out = act(LayerNorm(x) @ weight.T + bias)`` for ``count`` rows (``x[row_index]`` with
    a gather index): the norm into ``scratch`` (``[>= count, K]`` in the weight's dtype), then
    the product. Two kernels on purpose. A variant that computed the norm inside the few-rows
    product's kernel (statistics carried along by the kernel that last wrote the rows) was
    measured on a B200 in a 48-layer decode chain and lost at every row count, 59.7 against
    53.8 microseconds a layer at 8 rows: with programmatic dependent launch a kernel boundary
    costs less than the extra dependent phases inside the product's kernel."""
    if activation not in ACTIVATIONS:
        raise BackendError(f"linear_normed: unknown activation {activation!r}")
    layer_norm(x, gamma, beta, eps, scratch, rows=row_index, count=count)
    linear(scratch, weight, bias, out, activation=activation, rows=count)


def kv_store(k: torch.Tensor, v: torch.Tensor, slot_mapping: torch.Tensor,
             k_pages: torch.Tensor, v_pages: torch.Tensor, *, rows: int | None = None) -> None:
    """Write this step's key and value rows ``[N, kv_heads * head_dim]`` into the pages.

    Pages are ``[page, kv_head, slot, head_dim]``; ``slot_mapping[i] = page * page_size +
    slot`` or negative for a row that stores nothing. ``k`` and ``v`` share a row stride (they
    are column ranges of one projection output).
    """
    op = "kv_store"
    if _left_out and op in _left_out:
        return
    _need(op, "k", k, ndim=2)
    _need(op, "v", v, k.dtype, 2)
    _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
    _need(op, "k_pages", k_pages, k.dtype, 4)
    _need(op, "v_pages", v_pages, k.dtype, 4)
    if k.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    n = k.shape[0] if rows is None else rows
    if k.shape[1] != kv_heads * head_dim or v.shape != k.shape or k.stride(0) != v.stride(0) \
            or v_pages.shape != k_pages.shape or n > k.shape[0] or n > slot_mapping.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    fn = library("attention_simt").ayk_kv_store
    status = fn(_ptr(k), _ptr(v), c_int(k.stride(0)), _ptr(slot_mapping), _ptr(k_pages),
                _ptr(v_pages), c_int(n), c_int(kv_heads), c_int(head_dim), c_int(page_size),
                c_int(_TYPE[k.dtype]), _stream())
    check(status, op)


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              block_table: torch.Tensor, request_of_row: torch.Tensor, positions: torch.Tensor,
              out: torch.Tensor, *, num_heads: int, scale: float, window: int = 0,
              rows: int | None = None) -> None:
    """Causal attention of query rows over their requests' cached keys and values.

    ``q`` and ``out`` are ``[N, num_heads * head_dim]``; row ``i`` belongs to request
    ``request_of_row[i]`` (a row of ``block_table``; negative = padding row, output zero) and
    sits at ``positions[i]``; it sees keys ``max(0, p - window + 1) .. p`` (``window`` 0 = all).
    The keys of the step's own rows must already be stored.
    """
    op = "attention"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    n = q.shape[0] if rows is None else rows
    if q.shape[1] != num_heads * head_dim or out.shape[1] != q.shape[1] or n > out.shape[0] \
            or n > request_of_row.shape[0] or n > positions.shape[0] or \
            v_pages.shape != k_pages.shape:
        raise BackendError(f"{op}: shapes do not fit")
    fn = library("attention_simt").ayk_attention_simt
    status = fn(_ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(out),
                c_int(out.stride(0)), c_int(n), c_int(num_heads), c_int(kv_heads),
                c_int(head_dim), c_int(page_size), c_float(scale), c_int(window),
                c_int(_TYPE[q.dtype]), _stream())
    check(status, op)


#: Which kernel :func:`attention_prefill` launches for head size 64: ``"tcgen05"`` (both
#: products on the 5th-generation tensor cores, accumulators in tensor memory) or ``"mma"``
#: (the warp-level kernel that serves every other head size); tests switch it.
PREFILL_ATTENTION = "tcgen05"


def attention_prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, row_start: torch.Tensor, kv_len: torch.Tensor,
                      out: torch.Tensor, *, num_heads: int, scale: float, host_rows: list[int],
                      window: int = 0, kernel: str | None = None, keep_first: int = 0,
                      gate: torch.Tensor | None = None, pool: int = 0,
                      k_pool: torch.Tensor | None = None, v_pool: torch.Tensor | None = None,
                      sink: torch.Tensor | None = None) -> None:
    """Causal attention of prompt portions in bfloat16 on the tensor cores.

    Request ``b`` owns rows ``row_start[b] .. row_start[b + 1]`` of ``q`` and ``out``, which
    are the last rows of its ``kv_len[b]`` cached tokens; ``host_rows`` is the host copy of
    the row counts (the grid is sized from it). Head size 64 runs on tcgen05; the other head
    sizes on a warp-level kernel compiled for the head size (``kernel`` forces one of them).
    The warp-level kernel also takes value rows of another size than key rows (``v_pages``'
    last dimension), ``keep_first`` (with a window: keys before that position stay visible)
    and ``gate`` (float32 ``[N, num_heads * value size]``: the result times its sigmoid);
    with ``pool`` and a window the pooled rows ``k_pool`` / ``v_pool`` of the blocks that lie
    wholly behind a row's window (see :func:`pooled_attention`), and with ``sink`` (float32
    ``[num_heads]``) one more entry ``exp(sink[head])`` in the softmax's denominator.
    """
    op = "attention_prefill"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, torch.bfloat16, 2)
    _need(op, "out", out, torch.bfloat16, 2)
    _need(op, "k_pages", k_pages, torch.bfloat16, 4)
    _need(op, "v_pages", v_pages, torch.bfloat16, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "row_start", row_start, torch.int32, 1)
    _need(op, "kv_len", kv_len, torch.int32, 1)
    if not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    value_dim = v_pages.shape[3]
    count = len(host_rows)
    if q.shape[1] != num_heads * head_dim or out.shape[1] != num_heads * value_dim or \
            row_start.shape[0] < count + 1 or kv_len.shape[0] < count or \
            block_table.shape[0] < count or v_pages.shape[:3] != k_pages.shape[:3]:
        raise BackendError(f"{op}: shapes do not fit")
    if head_dim % 16 or not 16 <= head_dim <= 256 or value_dim % 16 or \
            not 16 <= value_dim <= 256:
        raise BackendError(f"{op}: head and value sizes must be multiples of 16 in [16, 256]")
    if gate is not None:
        _need(op, "gate", gate, torch.float32, 2)
        if gate.shape[1] != num_heads * value_dim or gate.stride(1) != 1:
            raise BackendError(f"{op}: the gate does not match the output")
    pooled = bool(pool and window)
    if pooled:
        _need(op, "k_pool", k_pool, torch.bfloat16, 4)
        _need(op, "v_pool", v_pool, torch.bfloat16, 4)
        slots = pool_slots(page_size, pool)
        if tuple(k_pool.shape) != (k_pages.shape[0], kv_heads, slots, head_dim) or \
                tuple(v_pool.shape) != (k_pages.shape[0], kv_heads, slots, value_dim) or \
                not k_pool.is_contiguous() or not v_pool.is_contiguous() or keep_first:
            raise BackendError(f"{op}: the pooled rows do not match the pages")
    if sink is not None:
        _need(op, "sink", sink, torch.float32, 1)
        if sink.shape[0] != num_heads:
            raise BackendError(f"{op}: one sink per head")
    plain = value_dim == head_dim and gate is None and not (keep_first and window) and \
        not pooled and sink is None
    # the tcgen05 kernel works on tiles of 256 rows: a step of short portions only is better
    # served by the warp-level kernel's tiles of 64
    which = kernel or (PREFILL_ATTENTION if head_dim == 64 and scale > 0 and plain
                       and max(host_rows, default=0) >= 256 else "mma")
    if which == "tcgen05":
        if head_dim != 64 or not plain:
            raise BackendError(f"{op}: the tcgen05 kernel serves head size 64 without a gate, "
                               f"kept keys or value rows of their own, not {head_dim}")
        lib = library("attention_prefill_tc")
        tile_rows = lib.ayk_attention_prefill_tc_rows()
        tiles = sum(-(-rows // tile_rows) for rows in host_rows)
        status = lib.ayk_attention_prefill_tc(
            _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
            c_int(block_table.stride(0)), _ptr(row_start), _ptr(kv_len), _ptr(out),
            c_int(out.stride(0)), c_int(count), c_int(tiles), c_int(num_heads), c_int(kv_heads),
            c_int(head_dim), c_int(page_size), c_int(k_pages.shape[0]), c_float(scale),
            c_int(window), _ptr(_status_word(q.device)), _stream())
        check(status, op)
        return
    tiles = sum(-(-rows // 64) for rows in host_rows)
    sizes = {"AYK_HEAD_DIM": head_dim}
    if value_dim != head_dim:
        sizes["AYK_VALUE_DIM"] = value_dim
    fn = library("attention_prefill", **sizes).ayk_attention_prefill_pooled
    status = fn(_ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                c_int(block_table.stride(0)), _ptr(row_start), _ptr(kv_len), _ptr(out),
                c_int(out.stride(0)), c_int(count), c_int(tiles), c_int(num_heads),
                c_int(kv_heads), c_int(head_dim), c_int(page_size), c_float(scale),
                c_int(window), c_int(value_dim), c_int(keep_first), _ptr(gate),
                c_int(0 if gate is None else gate.stride(0)),
                c_int(pool if pooled else 0), c_int(pool_slots(page_size, pool) if pooled else 0),
                _ptr(k_pool if pooled else None), _ptr(v_pool if pooled else None), _ptr(sink),
                _stream())
    check(status, op)


#: CTAs of the decode attention kernel the grid aims at per SM: six are resident (32 KB of
#: shared memory each), and a little over one round measured best
DECODE_CTAS_PER_SM = 7
_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """Streaming multiprocessors of ``device`` (the current one when absent), asked once."""
    index = torch.cuda.current_device() if device is None or device.index is None \
        else device.index
    found = _sm_counts.get(index)
    if found is None:
        found = torch.cuda.get_device_properties(index).multi_processor_count
        _sm_counts[index] = found
    return found


def decode_splits(num_rows: int, num_heads: int, max_kv_len: int,
                  device: torch.device | None = None) -> int:
    """How many CTAs share one (request, head) of a decode step: the grid should fill the
    device about once (``DECODE_CTAS_PER_SM`` CTAs per SM), a cluster merges up to 8 shares on
    chip, and a warp wants at least 32 keys."""
    fill = DECODE_CTAS_PER_SM * sm_count(device) // max(1, num_rows * num_heads)
    enough_keys = max(1, max_kv_len // 128)
    splits = max(1, min(fill, enough_keys, 8))
    while splits & (splits - 1):  # a power of two
        splits -= 1
    return splits


def attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, request_of_row: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, *, num_heads: int, scale: float,
                     window: int = 0, rows: int | None = None, splits: int = 1,
                     partial: torch.Tensor | None = None,
                     tickets: torch.Tensor | None = None, k_new: torch.Tensor | None = None,
                     v_new: torch.Tensor | None = None, store: bool = False) -> None:
    """Attention for steps whose every request brings one row (same contract as
    :func:`attention`). ``splits`` CTAs share each (request, head). Up to 8 splits merge on
    chip (a thread-block cluster); given ``partial`` (float32, at least rows * heads * splits
    * (head_dim + 2)) and ``tickets`` (int32 zeros, at least rows * heads; left zero) the
    shares go through that scratch instead, which more than 8 splits require. With ``k_new``/``v_new``
    (``[rows, kv_heads * head_dim]``, column ranges of the projection output) each row's own
    key and value are taken from there, and with ``store`` the kernel also writes them into
    the row's cache slot, so no separate KV store runs."""
    op = "attention_decode"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, head_dim = k_pages.shape
    n = q.shape[0] if rows is None else rows
    if q.shape[1] != num_heads * head_dim or out.shape[1] != q.shape[1] or n > out.shape[0] \
            or n > request_of_row.shape[0] or n > positions.shape[0] or \
            v_pages.shape != k_pages.shape:
        raise BackendError(f"{op}: shapes do not fit")
    if splits > 8 and partial is None:
        raise BackendError(f"{op}: more than 8 splits need scratch")
    if (partial is None) != (tickets is None):
        raise BackendError(f"{op}: partial and tickets come together")
    if partial is not None and tickets is not None:
        _need(op, "partial", partial, torch.float32)
        _need(op, "tickets", tickets, torch.int32)
        if partial.numel() < n * num_heads * splits * (head_dim + 2) or \
                tickets.numel() < n * num_heads:
            raise BackendError(f"{op}: the scratch buffers are too small")
    if k_new is not None:
        if v_new is None:
            raise BackendError(f"{op}: k_new needs v_new")
        _need(op, "k_new", k_new, q.dtype, 2)
        _need(op, "v_new", v_new, q.dtype, 2)
        if k_new.shape[1] != kv_heads * head_dim or v_new.shape != k_new.shape or \
                k_new.stride(0) != v_new.stride(0) or k_new.shape[0] < n:
            raise BackendError(f"{op}: k_new/v_new do not fit")
    elif store:
        raise BackendError(f"{op}: store needs k_new and v_new")
    status = library("attention_decode").ayk_attention_decode(
        _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(out),
        c_int(out.stride(0)), c_int(n), c_int(num_heads), c_int(kv_heads), c_int(head_dim),
        c_int(page_size), c_float(scale), c_int(window), c_int(splits), _ptr(partial),
        _ptr(tickets), _ptr(k_new), _ptr(v_new),
        c_int(0 if k_new is None else k_new.stride(0)), c_int(1 if store else 0),
        _ptr(_status_word(q.device)), c_int(_TYPE[q.dtype]), _stream(),
        c_int(k_pages.shape[0]))
    check(status, op)


ARGMAX_PARTS = 32


def argmax(logits: torch.Tensor, out: torch.Tensor, *, rows: int | None = None,
           scratch: torch.Tensor | None = None) -> None:
    """``out[i]`` = the id of row ``i``'s largest logit, the smallest id among equals.

    With ``scratch`` (float32, at least ``2 * rows * ARGMAX_PARTS`` elements) every row is
    split over ``ARGMAX_PARTS`` CTAs and folded by a second small kernel: faster for a few
    rows of a large vocabulary."""
    op = "argmax"
    if _left_out and op in _left_out:
        return
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "out", out, torch.int32, 1)
    n = logits.shape[0] if rows is None else rows
    if n > out.shape[0] or n > logits.shape[0]:
        raise BackendError(f"{op}: {n} rows do not fit")
    if scratch is not None:
        _need(op, "scratch", scratch, torch.float32)
        if scratch.numel() < 2 * n * ARGMAX_PARTS or not scratch.is_contiguous():
            raise BackendError(f"{op}: scratch is too small")
        flat = scratch.reshape(-1)
        values = flat[:n * ARGMAX_PARTS]
        ids = flat[n * ARGMAX_PARTS:2 * n * ARGMAX_PARTS].view(torch.int32)
        global _launches
        _launches += 1  # two kernels; _stream() below counts the other
        status = library("sampling").ayk_argmax_split(
            _ptr(logits), c_int(logits.stride(0)), c_int(n), c_int(logits.shape[1]),
            c_int(ARGMAX_PARTS), _ptr(values), _ptr(ids), _ptr(out), _stream())
        check(status, op)
        return
    status = library("sampling").ayk_argmax(_ptr(logits), c_int(logits.stride(0)), c_int(n),
                                            c_int(logits.shape[1]), _ptr(out), _stream())
    check(status, op)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor | None,
           top_p: torch.Tensor | None, min_p: torch.Tensor | None, seeds: torch.Tensor,
           positions: torch.Tensor, out: torch.Tensor, *, rows: int | None = None) -> None:
    """One token per row of fp32 logits: temperature, top-k, top-p, min-p and the inverse CDF
    over the canonical order, the random number from Philox(seed, position) in the kernel.

    ``temperature`` float32 (a row below 1e-5 is greedy); ``top_k`` int32 (<= 0 off);
    ``top_p``/``min_p`` float32; ``seeds``/``positions`` int64 (position = index in the
    sequence of the token being produced); ``out`` int32.
    """
    op = "sample"
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "temperature", temperature, torch.float32, 1)
    _need(op, "seeds", seeds, torch.int64, 1)
    _need(op, "positions", positions, torch.int64, 1)
    _need(op, "out", out, torch.int32, 1)
    n = logits.shape[0] if rows is None else rows
    for name, tensor, dtype in (("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                                ("min_p", min_p, torch.float32)):
        if tensor is not None:
            _need(op, name, tensor, dtype, 1)
            if tensor.shape[0] < n:
                raise BackendError(f"{op}: {name} has fewer than {n} rows")
    if min(temperature.shape[0], seeds.shape[0], positions.shape[0], out.shape[0],
           logits.shape[0]) < n:
        raise BackendError(f"{op}: {n} rows do not fit the tensors")
    status = library("sampling").ayk_sample(
        _ptr(logits), c_int(logits.stride(0)), c_int(n), c_int(logits.shape[1]),
        _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(positions),
        _ptr(out), _stream())
    check(status, op)


#: words of a row's header in the descriptor of :func:`logits_adjust`
ADJUST_WORDS = 16


def logits_scale_cap(logits: torch.Tensor, *, rows: int, scale: float = 1.0,
                     softcap: float = 0.0) -> None:
    """``x = scale * x`` and then, with ``softcap`` > 0, ``x = softcap * tanh(x / softcap)``
    on ``rows`` rows of fp32 ``logits`` in place (what some architectures do to the head's
    output; GPT-2 does neither and never launches this)."""
    op = "logits_scale_cap"
    _need(op, "logits", logits, torch.float32, 2)
    if rows < 0 or rows > logits.shape[0] or softcap < 0:
        raise BackendError(f"{op}: rows={rows}, softcap={softcap} do not fit")
    status = library("sampling").ayk_logits_scale_cap(
        _ptr(logits), c_int(logits.stride(0)), c_int(logits.shape[1]), c_int(rows),
        c_float(scale), c_float(softcap), _stream())
    check(status, op)


def logits_adjust(logits: torch.Tensor, desc: torch.Tensor, num_rows: int,
                  mask_scratch: torch.Tensor | None = None) -> None:
    """Adjust rows of fp32 ``logits`` in place before a token is chosen: allowed and banned
    ids, additive biases, repetition / frequency / presence penalties, in that order.

    ``desc`` (int32, on the device) holds ``num_rows`` headers of ``ADJUST_WORDS`` words
    followed by the lists they point to (offsets are word indices into ``desc``): row of
    ``logits``; history offset, history length, prompt length (the history is the request's
    prompt followed by its output); bias offset and count (ids, then as many float32 values);
    allowed offset and count (-1: no restriction); banned offset and count; repetition,
    frequency and presence as float32 bits. ``mask_scratch`` (int32, ``num_rows *
    ceil(vocab / 32)`` words) is needed when a row has an allowed list.
    """
    op = "logits_adjust"
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "desc", desc, torch.int32, 1)
    if num_rows < 0 or desc.shape[0] < num_rows * ADJUST_WORDS:
        raise BackendError(f"{op}: the descriptor does not hold {num_rows} rows")
    if mask_scratch is not None:
        _need(op, "mask_scratch", mask_scratch, torch.int32, 1)
        if mask_scratch.shape[0] < num_rows * ((logits.shape[1] + 31) // 32):
            raise BackendError(f"{op}: mask_scratch is too small")
    status = library("sampling").ayk_logits_adjust(
        _ptr(logits), c_int(logits.stride(0)), c_int(logits.shape[1]), _ptr(desc),
        c_int(num_rows), _ptr(mask_scratch), _stream())
    check(status, op)


# ---- norms by the root mean square, rotations ---------------------------------------------

GATES = {"none": 0, "silu_before": 1, "sigmoid_after": 2, "silu_after": 3}
ROPE_LAYOUTS = {"neighbours": 0, "halves": 1}


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
             weight_offset: float = 0.0, groups: int = 1, rows: torch.Tensor | None = None,
             count: int | None = None, gate: torch.Tensor | None = None,
             gate_mode: str = "none") -> None:
    """``out = x * rsqrt(mean(x^2) + eps) * (weight_offset + weight)`` over fp32 rows, the mean
    over each of ``groups`` equal parts of a row on its own; ``out`` float32 or bfloat16.

    With ``rows`` (int32), output row ``i`` normalises ``x[rows[i]]``. With ``gate`` (float32,
    laid out like ``x``): ``gate_mode="silu_before"`` multiplies ``x`` by ``silu(gate)`` before
    the norm, ``"sigmoid_after"`` multiplies the result by ``sigmoid(gate)``, ``"silu_after"``
    by ``silu(gate)``. A ``weight`` shorter than a row repeats along it (its length must divide
    a group's width: one weight shared by every head).
    """
    op = "rms_norm"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "weight", weight, torch.float32, 1)
    _need(op, "out", out, ndim=2)
    if out.dtype not in _TYPE:
        raise BackendError(f"{op}: out must be float32 or bfloat16, got {out.dtype}")
    width = out.shape[1]
    period = 0 if weight.shape[0] == width else weight.shape[0]
    if x.shape[1] != width or groups < 1 or width % groups or \
            (period and (width // groups) % period):
        raise BackendError(f"{op}: widths differ or {groups} groups do not divide {width}")
    if gate_mode not in GATES or (gate is None) != (gate_mode == "none"):
        raise BackendError(f"{op}: gate and gate_mode {gate_mode!r} do not go together")
    if gate is not None:
        _need(op, "gate", gate, torch.float32, 2)
        if gate.shape[1] != width or gate.shape[0] < x.shape[0]:
            raise BackendError(f"{op}: the gate does not match x")
    if rows is not None:
        _need(op, "rows", rows, torch.int32, 1)
    n = count if count is not None else (rows.shape[0] if rows is not None else x.shape[0])
    if n > out.shape[0] or (rows is None and n > x.shape[0]) or \
            (rows is not None and n > rows.shape[0]):
        raise BackendError(f"{op}: {n} rows do not fit the tensors")
    status = library("rms_norm").ayk_rms_norm(
        _ptr(x), c_int(x.stride(0)), _ptr(rows), _ptr(weight), c_float(weight_offset),
        c_float(eps), c_int(groups), _ptr(gate), c_int(0 if gate is None else gate.stride(0)),
        c_int(GATES[gate_mode]), _ptr(out), c_int(out.stride(0)), c_int(n), c_int(width),
        c_int(_TYPE[out.dtype]), c_int(period), _stream())
    check(status, op)


def rope_frequencies(dims: int, base: float, device: torch.device,
                     scaling: tuple[float, float, float, float] | None = None) -> torch.Tensor:
    """``f_i = base^(-2i / dims)`` for the ``dims / 2`` pairs, as float64 on ``device`` (the
    kernels form ``position * f_i`` and its sine and cosine in double precision).

    ``scaling = (factor, low, high, original)`` rescales by wavelength ``l = 2 pi / f``: a
    pair with ``l > original / low`` turns ``factor`` times slower, one with ``l < original /
    high`` is kept, and between the two the slowed and the kept frequency are blended with
    the weight ``(original / l - low) / (high - low)`` on the kept one."""
    values = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = scaling
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                keep = (original / wavelength - low) / (high - low)
                f = (1.0 - keep) * f / factor + keep * f
        values.append(f)
    return torch.tensor(values, dtype=torch.float64, device=device)


def rope(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, *, heads: int,
         head_stride: int, offset: int = 0, layout: str = "neighbours",
         rows: int | None = None) -> None:
    """Rotary position encoding in place: in each of the ``heads`` stretches of
    ``head_stride`` values of a row, the ``2 * len(freq)`` entries from ``offset`` on are
    rotated by ``positions[row] * freq[i]``: pair ``i`` is entries ``(2i, 2i+1)``
    (``"neighbours"``) or ``(i, i + dims/2)`` (``"halves"``)."""
    op = "rope"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, ndim=2)
    _need(op, "positions", positions, torch.int32, 1)
    _need(op, "freq", freq, torch.float64, 1)
    if x.dtype not in _TYPE or layout not in ROPE_LAYOUTS:
        raise BackendError(f"{op}: float32 or bfloat16 rows and a known layout only")
    n = x.shape[0] if rows is None else rows
    if n > x.shape[0] or n > positions.shape[0] or heads * head_stride > x.shape[1]:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("rope").ayk_rope(
        _ptr(x), c_int(x.stride(0)), _ptr(positions), _ptr(freq), c_int(n), c_int(heads),
        c_int(head_stride), c_int(offset), c_int(2 * freq.shape[0]), c_int(ROPE_LAYOUTS[layout]),
        c_int(_TYPE[x.dtype]), _stream())
    check(status, op)


# ---- latent attention -----------------------------------------------------------------------

def latent_prepare(proj: torch.Tensor, *, kv_offset: int, latent_weight: torch.Tensor,
                   eps: float, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                   freq: torch.Tensor, layout: str, pages: torch.Tensor | None,
                   q_plain: torch.Tensor, qa: torch.Tensor, heads: int, dim: int, rot: int,
                   rank: int, rows: int) -> None:
    """From a row of the fused projection (float32: the heads' queries ``[dim | rot]``, then
    at ``kv_offset`` the raw latent of ``rank`` entries and the raw shared key piece of
    ``rot``): the latent normalised by its root mean square times ``latent_weight`` and the
    rotated key piece go to the row's cache slot (``pages`` ``[page, 1, slot, rank + rot]``),
    the unrotated query parts to ``q_plain`` ``[N, heads * dim]``, the rotated ones to
    ``qa[:, h, rank:]`` (``qa`` is ``[N, heads * (rank + rot)]``). Without ``pages`` (a layer
    that reads latents another layer stored) the columns from ``kv_offset`` on are not read."""
    op = "latent_prepare"
    if _left_out and op in _left_out:
        return
    _need(op, "proj", proj, torch.float32, 2)
    _need(op, "latent_weight", latent_weight, torch.float32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    _need(op, "freq", freq, torch.float64, 1)
    _need(op, "q_plain", q_plain, ndim=2)
    _need(op, "qa", qa, q_plain.dtype, 2)
    if q_plain.dtype not in _TYPE or layout not in ROPE_LAYOUTS:
        raise BackendError(f"{op}: float32 or bfloat16 and a known layout only")
    if pages is not None:
        _need(op, "pages", pages, q_plain.dtype, 4)
        if slot_mapping is None or not pages.is_contiguous() or pages.shape[1] != 1 or \
                pages.shape[3] != rank + rot:
            raise BackendError(f"{op}: pages must be contiguous [page, 1, slot, rank + rot] "
                               "and come with a slot mapping")
        _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
    if rows > proj.shape[0] or rows > positions.shape[0] or rows > q_plain.shape[0] or \
            rows > qa.shape[0] or latent_weight.shape[0] != rank or \
            q_plain.shape[1] != heads * dim or qa.shape[1] != heads * (rank + rot) or \
            (pages is not None and proj.shape[1] < kv_offset + rank + rot) or \
            proj.shape[1] < heads * (dim + rot) or \
            (slot_mapping is not None and rows > slot_mapping.shape[0]):
        raise BackendError(f"{op}: shapes do not fit")
    status = library("latent_attention").ayk_latent_prepare(
        _ptr(proj), c_int(proj.stride(0)), c_int(kv_offset), _ptr(latent_weight), c_float(eps),
        _ptr(positions), _ptr(slot_mapping if pages is not None else None), _ptr(freq),
        c_int(2 * freq.shape[0]), c_int(ROPE_LAYOUTS[layout]), _ptr(pages), _ptr(q_plain),
        c_int(q_plain.stride(0)), _ptr(qa), c_int(qa.stride(0)), c_int(rows), c_int(heads),
        c_int(dim), c_int(rot), c_int(rank), c_int(_TYPE[q_plain.dtype]), _stream())
    check(status, op)


def head_linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, *, heads: int,
                transposed: bool, rows: int, gate: torch.Tensor | None = None,
                inner: int | None = None) -> None:
    """One small product per head, fp32 sums in a fixed order.

    ``a`` is ``[N, heads * I']`` of which a head's first ``I = inner`` columns are used
    (all ``I'`` when absent), and ``out`` ``[N, heads * J']`` with ``J' >= J`` (a head's
    results start every ``out.shape[1] / heads`` columns). ``weight`` holds the heads' matrices
    one under the other: ``[heads * J, I]`` applied as ``W_h a_h`` (``transposed=False``), or
    ``[heads * I, J]`` applied as ``W_h^T a_h`` (``transposed=True``). With ``gate`` (float32
    ``[N, heads * J]``) the result is multiplied by ``sigmoid(gate)``."""
    op = "head_linear"
    if _left_out and op in _left_out:
        return
    _need(op, "a", a, ndim=2)
    _need(op, "weight", weight, a.dtype, 2)
    _need(op, "out", out, a.dtype, 2)
    if a.dtype not in _TYPE or not weight.is_contiguous():
        raise BackendError(f"{op}: float32 or bfloat16 and a contiguous weight only")
    if heads < 1 or a.shape[1] % heads or out.shape[1] % heads or weight.shape[0] % heads:
        raise BackendError(f"{op}: {heads} heads do not divide the widths")
    a_head = a.shape[1] // heads
    inner = a_head if inner is None else inner
    if not 1 <= inner <= a_head:
        raise BackendError(f"{op}: a head of a has {a_head} columns, not {inner}")
    if transposed:
        if weight.shape[0] // heads != inner:
            raise BackendError(f"{op}: the weight's rows per head are not a's columns per head")
        outer, w_in, w_out = weight.shape[1], weight.shape[1], 1
    else:
        if weight.shape[1] != inner:
            raise BackendError(f"{op}: the weight's columns are not a's columns per head")
        outer, w_in, w_out = weight.shape[0] // heads, 1, weight.shape[1]
    out_head = out.shape[1] // heads
    if outer > out_head or rows > a.shape[0] or rows > out.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    if gate is not None:
        _need(op, "gate", gate, torch.float32, 2)
        if gate.shape[1] != heads * outer or gate.shape[0] < rows:
            raise BackendError(f"{op}: the gate does not match the result")
    status = library("latent_attention").ayk_head_linear(
        _ptr(a), c_int(a.stride(0)), c_int(a_head), _ptr(weight),
        c_longlong(weight.shape[0] // heads * weight.shape[1]), c_int(w_in), c_int(w_out),
        _ptr(gate), c_int(0 if gate is None else gate.stride(0)), _ptr(out),
        c_int(out.stride(0)), c_int(out_head), c_int(rows), c_int(heads), c_int(inner),
        c_int(outer), c_int(_TYPE[a.dtype]), _stream())
    check(status, op)


def latent_attention(qa: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     request_of_row: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                     *, num_heads: int, rank: int, scale: float, window: int = 0,
                     rows: int | None = None) -> None:
    """Attention of all heads over one latent row per token: the row of request
    ``request_of_row[i]`` at ``positions[i]`` scores ``scale * qa[i, h] . page_row`` over keys
    ``max(0, p - window + 1) .. p`` (``window`` 0: all) and returns the softmax-weighted sum of
    the page rows' first ``rank`` entries: ``out`` is ``[N, num_heads * rank]``. ``pages`` is
    ``[page, 1, slot, rank + rot]``; the step's own rows must already be stored."""
    op = "latent_attention"
    if _left_out and op in _left_out:
        return
    _need(op, "qa", qa, ndim=2)
    _need(op, "out", out, qa.dtype, 2)
    _need(op, "pages", pages, qa.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if qa.dtype not in _TYPE or not pages.is_contiguous() or pages.shape[1] != 1:
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages [page, 1, slot, row]")
    _, _, page_size, key_dim = pages.shape
    n = qa.shape[0] if rows is None else rows
    if qa.shape[1] != num_heads * key_dim or out.shape[1] != num_heads * rank or \
            rank > key_dim or n > out.shape[0] or n > request_of_row.shape[0] or \
            n > positions.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("latent_attention").ayk_latent_attention(
        _ptr(qa), c_int(qa.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(out),
        c_int(out.stride(0)), c_int(n), c_int(num_heads), c_int(rank), c_int(key_dim - rank),
        c_int(page_size), c_float(scale), c_int(window), c_int(_TYPE[qa.dtype]), _stream())
    check(status, op)


def set_latent_decode_tensor_cores(enabled: bool) -> None:
    """Let :func:`latent_decode` run bfloat16 steps on the warp-level tensor cores where the
    sizes allow (the default), or keep every call on its CUDA-core kernel (tests of that
    kernel, measurements of one against the other)."""
    library("latent_attention").ayk_set_latent_decode_tensor_cores(c_int(1 if enabled else 0))


def latent_decode_splits(rows: int, num_heads: int, reach: int,
                         device: torch.device | None = None) -> int:
    """Shares a row's keys are cut into by :func:`latent_decode`: about one CTA per SM over
    all rows, at least four tiles of 32 keys a share (one for each warp of the tensor-core
    kernel), and no share left without tiles (a share is ``ceil(tiles / shares)`` tiles, so
    the count is rounded to what that fills)."""
    tiles = reach // 32 + 2
    groups = -(-num_heads // 16)
    want = max(1, min(sm_count(device) // max(1, rows * groups), 64))
    per = max(4, -(-tiles // want))
    return max(1, min(-(-tiles // per), 64))


def latent_decode(qa: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                  request_of_row: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                  partial: torch.Tensor, *, num_heads: int, rank: int, scale: float,
                  window: int, rows: int, splits: int) -> bool:
    """:func:`latent_attention` for steps of single rows: one CTA per (row, share of its
    keys) serves every head, so a latent row leaves memory once. A head's result lands in the
    first ``rank`` of its ``out.shape[1] / num_heads`` columns. ``partial`` is float32 scratch
    of at least ``rows * num_heads * splits * (rank + 2)`` elements. Returns False, having
    run nothing, for sizes the kernel does not take."""
    op = "latent_decode"
    if _left_out and op in _left_out:
        return True
    _need(op, "qa", qa, ndim=2)
    _need(op, "out", out, qa.dtype, 2)
    _need(op, "pages", pages, qa.dtype, 4)
    _need(op, "partial", partial, torch.float32)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if qa.dtype not in _TYPE or not pages.is_contiguous() or pages.shape[1] != 1 or \
            not partial.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages [page, 1, slot, row]")
    _, _, page_size, key_dim = pages.shape
    if qa.shape[1] != num_heads * key_dim or out.shape[1] % num_heads or \
            out.shape[1] // num_heads < rank or rank > key_dim or rows > out.shape[0] or \
            rows > qa.shape[0] or rows > request_of_row.shape[0] or \
            rows > positions.shape[0] or \
            partial.numel() < rows * num_heads * splits * (rank + 2):
        raise BackendError(f"{op}: shapes do not fit")
    global _launches
    status = library("latent_attention").ayk_latent_decode(
        _ptr(qa), c_int(qa.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(partial),
        _ptr(out), c_int(out.stride(0)), c_int(out.shape[1] // num_heads), c_int(rows),
        c_int(num_heads), c_int(rank), c_int(key_dim - rank), c_int(page_size), c_float(scale),
        c_int(window), c_int(splits), c_int(_TYPE[qa.dtype]), _stream())
    if status == -6:  # AYK_NOT_TAKEN
        _launches -= 1
        return False
    _launches += 1  # the merge of the shares is a launch of its own
    check(status, op)
    return True


# ---- layers with a running state ------------------------------------------------------------

#: columns of a matrix state that one CTA of the scan kernels owns (``SCAN_COLS`` in
#: ``csrc/recurrent.cu``); the mLSTM state keeps its normaliser and maximum once per such tile
SCAN_COLUMNS = 16


def scan_state_floats(kind: str, *, heads: int, inner: int, columns: int, taps: int = 1,
                      channels: int = 0) -> int:
    """Floats of one request's state: ``"mamba2"``: the ``taps - 1`` kept inputs of
    ``channels`` channels, then ``heads`` matrices ``[inner, columns]``; ``"mlstm"``: ``heads``
    matrices ``[inner, columns]``, then a normaliser ``[inner]`` and a maximum per head and
    tile of ``SCAN_COLUMNS`` columns."""
    matrices = heads * inner * columns
    if kind == "mamba2":
        return (taps - 1) * channels + matrices
    if kind == "mlstm":
        tiles = -(-columns // SCAN_COLUMNS)
        return matrices + heads * tiles * (inner + 1)
    raise BackendError(f"scan_state_floats: unknown kind {kind!r}")


def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                     state: torch.Tensor, out: torch.Tensor, *, request_of_row: torch.Tensor,
                     row_start: torch.Tensor, state_slot: torch.Tensor, rows: int,
                     requests: int) -> None:
    """``out = silu(bias + causal convolution of x per channel)`` for the step's rows
    (float32 ``[N, channels]``; ``weight`` ``[channels, taps]``, its last column the current
    row's), with the ``taps - 1`` inputs before each request's first row taken from
    ``state[slot, :(taps - 1) * channels]``, which is then moved on to the step's end."""
    op = "causal_conv_silu"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "weight", weight, torch.float32, 2)
    _need(op, "state", state, torch.float32, 2)
    _need(op, "out", out, torch.float32, 2)
    channels, taps = weight.shape
    if bias is not None:
        _need(op, "bias", bias, torch.float32, 1)
    if x.shape[1] != channels or out.shape[1] != channels or rows > x.shape[0] or \
            rows > out.shape[0] or state.shape[1] < (taps - 1) * channels or \
            not weight.is_contiguous() or (bias is not None and bias.shape[0] != channels):
        raise BackendError(f"{op}: shapes do not fit")
    global _launches
    _launches += 1 if taps > 1 else 0  # the update of the kept inputs is a launch of its own
    status = library("recurrent").ayk_causal_conv_silu(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(bias), _ptr(state),
        c_longlong(state.stride(0)), _ptr(request_of_row), _ptr(row_start), _ptr(state_slot),
        _ptr(out), c_int(out.stride(0)), c_int(rows), c_int(requests), c_int(channels),
        c_int(taps), _stream())
    check(status, op)


def mamba2_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor,
                a_log: torch.Tensor, skip: torch.Tensor | None, state: torch.Tensor,
                y: torch.Tensor, *, row_start: torch.Tensor, state_slot: torch.Tensor,
                requests: int, heads: int, groups: int, state_size: int, columns: int) -> None:
    """The state-space recurrence over each request's rows. ``xbc`` float32
    ``[N, heads * columns + 2 * groups * state_size]`` (x, then B, then C, after convolution
    and activation), ``dt_raw`` ``[N, heads]``; per head ``S <- exp(-exp(a_log) dt) S + dt B
    x^T``, ``y = S^T C + skip * x`` with ``dt = softplus(dt_raw + dt_bias)``. ``state``
    ``[slots, heads * state_size * columns]`` (a view of the matrices' part of the state)."""
    op = "mamba2_scan"
    if _left_out and op in _left_out:
        return
    for name, tensor in (("xbc", xbc), ("dt_raw", dt_raw), ("state", state), ("y", y)):
        _need(op, name, tensor, torch.float32, 2)
    for name, tensor in (("dt_bias", dt_bias), ("a_log", a_log)):
        _need(op, name, tensor, torch.float32, 1)
        if tensor.shape[0] != heads:
            raise BackendError(f"{op}: {name} must have one entry per head")
    if xbc.shape[1] != heads * columns + 2 * groups * state_size or dt_raw.shape[1] != heads or \
            y.shape[1] != heads * columns or state.shape[1] < heads * state_size * columns:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("recurrent").ayk_mamba2_scan(
        _ptr(xbc), c_int(xbc.stride(0)), _ptr(dt_raw), c_int(dt_raw.stride(0)), _ptr(dt_bias),
        _ptr(a_log), _ptr(skip), _ptr(state), c_longlong(state.stride(0)), _ptr(row_start),
        _ptr(state_slot), _ptr(y), c_int(y.stride(0)), c_int(requests), c_int(heads),
        c_int(groups), c_int(state_size), c_int(columns), _stream())
    check(status, op)


def mlstm_scan(proj: torch.Tensor, gate_bias: torch.Tensor | None, state: torch.Tensor,
               out: torch.Tensor, *, row_start: torch.Tensor, state_slot: torch.Tensor,
               requests: int, heads: int, dim: int, columns: int, k_offset: int, v_offset: int,
               i_offset: int, f_offset: int, cap: float) -> None:
    """The matrix-memory recurrence over each request's rows. ``proj`` float32 rows hold the
    queries at 0, keys at ``k_offset`` (``heads * dim`` each), values at ``v_offset``
    (``heads * columns``) and the raw input and forget gates at ``i_offset`` / ``f_offset``
    (``heads`` each); ``gate_bias`` ``[2 * heads]`` (input, then forget). ``out``
    ``[N, heads * columns]`` is the memory's answer before norm and output gate. ``state``
    ``[slots, scan_state_floats("mlstm", ...)]``."""
    op = "mlstm_scan"
    if _left_out and op in _left_out:
        return
    for name, tensor in (("proj", proj), ("state", state), ("out", out)):
        _need(op, name, tensor, torch.float32, 2)
    if gate_bias is not None:
        _need(op, "gate_bias", gate_bias, torch.float32, 1)
    need = scan_state_floats("mlstm", heads=heads, inner=dim, columns=columns)
    if state.shape[1] < need or out.shape[1] != heads * columns or \
            proj.shape[1] < max(k_offset + heads * dim, v_offset + heads * columns,
                                i_offset + heads, f_offset + heads) or \
            (gate_bias is not None and gate_bias.shape[0] != 2 * heads):
        raise BackendError(f"{op}: shapes do not fit")
    status = library("recurrent").ayk_mlstm_scan(
        _ptr(proj), c_int(proj.stride(0)), c_int(k_offset), c_int(v_offset), c_int(i_offset),
        c_int(f_offset), _ptr(gate_bias), c_float(cap), _ptr(state),
        c_longlong(state.stride(0)), _ptr(row_start), _ptr(state_slot), _ptr(out),
        c_int(out.stride(0)), c_int(requests), c_int(heads), c_int(dim), c_int(columns),
        _stream())
    check(status, op)


def gla_scan(proj: torch.Tensor, decay_raw: torch.Tensor, state: torch.Tensor,
             out: torch.Tensor, *, row_start: torch.Tensor, state_slot: torch.Tensor,
             requests: int, heads: int, dim: int, columns: int, k_offset: int, v_offset: int,
             tau: float, q_scale: float) -> None:
    """Gated linear attention with a decay per key channel over each request's rows. ``proj``
    float32 rows hold the queries at 0, keys at ``k_offset`` (``heads * dim`` each) and values
    at ``v_offset`` (``heads * columns``); ``decay_raw`` ``[N, heads * dim]`` the raw decays
    ``z``. Per head ``S <- diag(sigmoid(z)^(1/tau)) S + k v^T`` (the decay of key channel ``n``
    on row ``n`` of ``S``) and ``out = q_scale * S^T q``. ``state`` ``[slots, heads * dim *
    columns]`` float32, a slot's ``S`` kept as ``[heads][columns][dim]``."""
    op = "gla_scan"
    if _left_out and op in _left_out:
        return
    for name, tensor in (("proj", proj), ("decay_raw", decay_raw), ("state", state),
                         ("out", out)):
        _need(op, name, tensor, torch.float32, 2)
    if state.shape[1] < heads * dim * columns or out.shape[1] != heads * columns or \
            decay_raw.shape[1] != heads * dim or \
            proj.shape[1] < max(k_offset + heads * dim, v_offset + heads * columns):
        raise BackendError(f"{op}: shapes do not fit")
    status = library("recurrent").ayk_gla_scan(
        _ptr(proj), c_int(proj.stride(0)), c_int(k_offset), c_int(v_offset), _ptr(decay_raw),
        c_int(decay_raw.stride(0)), c_float(tau), c_float(q_scale), _ptr(state),
        c_longlong(state.stride(0)), _ptr(row_start), _ptr(state_slot), _ptr(out),
        c_int(out.stride(0)), c_int(requests), c_int(heads), c_int(dim), c_int(columns),
        _stream())
    check(status, op)


# ---- attention with mixed heads, mixers side by side ----------------------------------------

def talking_prepare(proj: torch.Tensor, *, k_offset: int, v_offset: int,
                    bias: torch.Tensor | None, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                    positions: torch.Tensor, freq: torch.Tensor | None, layout: str,
                    talk: torch.Tensor | None, temp: torch.Tensor | None, scale: float,
                    slot_mapping: torch.Tensor | None, k_pages: torch.Tensor | None,
                    v_pages: torch.Tensor | None, qmix: torch.Tensor, heads: int, kv_heads: int,
                    dim: int, vdim: int, rows: int) -> None:
    """From a row of a fused projection (float32: ``heads * dim`` queries at 0, ``kv_heads *
    dim`` keys at ``k_offset``, ``kv_heads * vdim`` values at ``v_offset``): queries and keys
    each normalised by the root mean square over their whole projection with a weight per
    entry (``q_weight`` / ``k_weight``; ``None``: no norm) after ``bias`` (float32, laid out as
    the projection's query, key and value columns; optional) is added, the first ``2 * len(freq)`` entries
    of every head rotated by the position, the key and value stored into the row's cache
    slot (``k_pages`` ``[page, kv_head, slot, dim]``, ``v_pages`` likewise with ``vdim``), and
    the *mixed queries* written to ``qmix`` ``[N, heads * kv_heads * dim]``:
    ``m[h, g] = sum over heads a of group g of talk[h, a] * temp[a] * scale * q[a]``, so that
    head ``h``'s mixed score against a token is ``sum_g m[h, g] . k[g]``."""
    op = "talking_prepare"
    if _left_out and op in _left_out:
        return
    _need(op, "proj", proj, torch.float32, 2)
    _need(op, "positions", positions, torch.int32, 1)
    _need(op, "qmix", qmix, ndim=2)
    if qmix.dtype not in _TYPE or layout not in ROPE_LAYOUTS:
        raise BackendError(f"{op}: float32 or bfloat16 and a known layout only")
    for name, tensor, size in (("bias", bias, v_offset + kv_heads * vdim),
                               ("q_weight", q_weight, heads * dim),
                               ("k_weight", k_weight, kv_heads * dim),
                               ("talk", talk, heads * heads), ("temp", temp, heads)):
        if tensor is not None:
            _need(op, name, tensor, torch.float32)
            if tensor.numel() != size or not tensor.is_contiguous():
                raise BackendError(f"{op}: {name} must hold {size} contiguous entries")
    page_size = 1
    if k_pages is not None:
        if v_pages is None or slot_mapping is None:
            raise BackendError(f"{op}: key pages come with value pages and a slot mapping")
        _need(op, "k_pages", k_pages, qmix.dtype, 4)
        _need(op, "v_pages", v_pages, qmix.dtype, 4)
        _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
        page_size = k_pages.shape[2]
        if tuple(k_pages.shape[1:]) != (kv_heads, page_size, dim) or \
                tuple(v_pages.shape[1:]) != (kv_heads, page_size, vdim) or \
                not k_pages.is_contiguous() or not v_pages.is_contiguous() or \
                rows > slot_mapping.shape[0]:
            raise BackendError(f"{op}: pages must be contiguous [page, kv_head, slot, dim]")
    rot_dims = 0
    if freq is not None and freq.numel():
        _need(op, "freq", freq, torch.float64, 1)
        rot_dims = 2 * freq.shape[0]
    if rows > proj.shape[0] or rows > positions.shape[0] or rows > qmix.shape[0] or \
            qmix.shape[1] != heads * kv_heads * dim or \
            proj.shape[1] < v_offset + kv_heads * vdim:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("talking_attention").ayk_talking_prepare(
        _ptr(proj), c_int(proj.stride(0)), c_int(k_offset), c_int(v_offset), _ptr(bias),
        _ptr(q_weight), _ptr(k_weight), c_float(eps), _ptr(positions), _ptr(freq if rot_dims else None),
        c_int(rot_dims), c_int(ROPE_LAYOUTS[layout]), _ptr(talk), _ptr(temp), c_float(scale),
        _ptr(slot_mapping if k_pages is not None else None), _ptr(k_pages), _ptr(v_pages),
        c_int(page_size), _ptr(qmix), c_int(qmix.stride(0)), c_int(rows), c_int(heads),
        c_int(kv_heads), c_int(dim), c_int(vdim), c_int(_TYPE[qmix.dtype]), _stream())
    check(status, op)


def talking_attention(qmix: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, request_of_row: torch.Tensor,
                      positions: torch.Tensor, out: torch.Tensor, *, heads: int, chunk: int = 0,
                      window: int = 0, reach: int, gate: torch.Tensor | None = None,
                      rows: int | None = None, single_rows: bool = False,
                      tensor_cores: bool = True) -> None:
    """Softmax attention of mixed queries (see :func:`talking_prepare`; every factor is in
    them) over paged keys and values. The row of request ``request_of_row[i]`` at
    ``positions[i]`` sees the keys from the start of its block of ``chunk`` positions
    (``chunk`` 0: from 0), and no further back than ``window`` (0: no limit), up to itself;
    head ``h`` sums the values of key/value head ``h // (heads / kv_heads)``; with ``gate``
    (float32 ``[N, heads]``) its result is multiplied by ``sigmoid(gate[:, h])``. ``reach``
    bounds the keys any row sees. The step's own keys must already be stored. bfloat16 runs
    on the warp-level tensor cores where the sizes allow (``tensor_cores=False``: never), with
    a CTA per row when ``single_rows`` says that every request brings one row, else per 16
    rows; float32 on the CUDA cores."""
    op = "talking_attention"
    if _left_out and op in _left_out:
        return
    _need(op, "qmix", qmix, ndim=2)
    _need(op, "out", out, qmix.dtype, 2)
    _need(op, "k_pages", k_pages, qmix.dtype, 4)
    _need(op, "v_pages", v_pages, qmix.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if qmix.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    n = qmix.shape[0] if rows is None else rows
    if qmix.shape[1] != heads * kv_heads * dim or out.shape[1] != heads * vdim or \
            tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3]) or n > out.shape[0] or \
            n > request_of_row.shape[0] or n > positions.shape[0] or heads % kv_heads:
        raise BackendError(f"{op}: shapes do not fit")
    if gate is not None:
        _need(op, "gate", gate, torch.float32, 2)
        if gate.shape[1] != heads or gate.shape[0] < n:
            raise BackendError(f"{op}: the gate does not match the rows")
    status = library("talking_attention").ayk_talking_attention(
        _ptr(qmix), c_int(qmix.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(gate),
        c_int(0 if gate is None else gate.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(n),
        c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(page_size), c_int(chunk),
        c_int(window), c_int(max(1, reach)),
        c_int(0 if not tensor_cores else (1 if single_rows else 16)), c_int(_TYPE[qmix.dtype]),
        _stream())
    check(status, op)


def norm_sum(branches: list[torch.Tensor], weights: list[torch.Tensor], eps: float,
             dst: torch.Tensor, *, factor: float, scale: torch.Tensor | None = None,
             accumulate: bool = True, rows: int) -> None:
    """``dst (+)= scale * factor * sum_b rms_norm(branches[b]) * weights[b]``: up to four
    float32 ``[N, width]`` results, each normalised over the whole width by its root mean
    square with its own weight, summed, multiplied element by element by ``scale`` (float32
    ``[width]``, optional) and added to (``accumulate``) or written into float32 ``dst``."""
    op = "norm_sum"
    if _left_out and op in _left_out:
        return
    _need(op, "dst", dst, torch.float32, 2)
    width = dst.shape[1]
    if len(branches) != len(weights) or not 1 <= len(branches) <= 4 or rows > dst.shape[0]:
        raise BackendError(f"{op}: one weight per branch, one to four branches")
    for branch, weight in zip(branches, weights):
        _need(op, "branch", branch, torch.float32, 2)
        _need(op, "weight", weight, torch.float32, 1)
        if branch.shape[1] != width or weight.shape[0] != width or rows > branch.shape[0]:
            raise BackendError(f"{op}: widths differ")
    if scale is not None:
        _need(op, "scale", scale, torch.float32, 1)
        if scale.shape[0] != width:
            raise BackendError(f"{op}: the scale does not match the width")
    count = len(branches)
    xs = (c_void_p * count)(*[b.data_ptr() for b in branches])
    ws = (c_void_p * count)(*[w.data_ptr() for w in weights])
    lds = (c_int * count)(*[b.stride(0) for b in branches])
    status = library("rms_norm").ayk_norm_sum(
        xs, lds, ws, c_int(count), c_float(eps), c_float(factor), _ptr(scale), _ptr(dst),
        c_int(dst.stride(0)), c_int(rows), c_int(width), c_int(1 if accumulate else 0),
        _stream())
    check(status, op)


def scale_add(x: torch.Tensor, scale: torch.Tensor, dst: torch.Tensor, *, rows: int,
              accumulate: bool = True) -> None:
    """``dst (+)= scale * x`` over float32 rows, ``scale`` a float32 vector of the width."""
    op = "scale_add"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "scale", scale, torch.float32, 1)
    _need(op, "dst", dst, torch.float32, 2)
    width = dst.shape[1]
    if x.shape[1] != width or scale.shape[0] != width or rows > x.shape[0] or \
            rows > dst.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("rms_norm").ayk_scale_add(
        _ptr(x), c_int(x.stride(0)), _ptr(scale), _ptr(dst), c_int(dst.stride(0)), c_int(rows),
        c_int(width), c_int(1 if accumulate else 0), _stream())
    check(status, op)


# ---- mixture of experts ---------------------------------------------------------------------

#: pairs (row, chosen expert) per tile of the grouped products (``MOE_TM`` in ``csrc/moe.cu``),
#: and per tile of the bfloat16 products of steps with many rows (``MOE_TM_WIDE``)
MOE_TILE_ROWS = 32
MOE_TILE_ROWS_WIDE = 128


def moe_max_tiles(rows: int, experts: int, top: int, tile_rows: int = MOE_TILE_ROWS) -> int:
    """Tiles the grouped products may need for ``rows`` rows: every expert's pairs are padded
    to whole tiles."""
    pairs = rows * top
    return -(-(pairs + min(experts, pairs) * (tile_rows - 1)) // tile_rows)


def moe_tile_rows(rows: int, experts: int, top: int, dtype: torch.dtype) -> int:
    """Rows of a tile :func:`moe_experts` uses: the wide tile in bfloat16 once an expert gets
    two narrow tiles' worth of pairs on average, else the narrow one."""
    wide = dtype == torch.bfloat16 and rows * top >= 2 * MOE_TILE_ROWS * experts
    return MOE_TILE_ROWS_WIDE if wide else MOE_TILE_ROWS


def moe_scratch(rows: int, experts: int, top: int) -> tuple[int, int]:
    """``(places, tiles)``: the most rows of ``sorted_pairs`` / ``inner`` and the most entries
    of ``tile_expert`` any tile size needs for up to ``rows`` rows."""
    sizes = (MOE_TILE_ROWS, MOE_TILE_ROWS_WIDE)
    return (max(moe_max_tiles(rows, experts, top, t) * t for t in sizes),
            max(moe_max_tiles(rows, experts, top, t) for t in sizes))


def moe_route(logits: torch.Tensor, chosen: torch.Tensor, share: torch.Tensor, *, top: int,
              rows: int, over_all: bool = False) -> None:
    """Per row of float32 ``logits`` ``[N, experts]``: the ``top`` largest (ties to the smaller
    index), in descending order, into ``chosen`` (int32 ``[N * top]``), and the softmax over
    just those into ``share`` (float32 ``[N * top]``); with ``over_all`` the chosen ones' part
    of the softmax over every expert instead (shares that do not add up to one)."""
    op = "moe_route"
    if _left_out and op in _left_out:
        return
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "chosen", chosen, torch.int32, 1)
    _need(op, "share", share, torch.float32, 1)
    if rows > logits.shape[0] or min(chosen.shape[0], share.shape[0]) < rows * top:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("moe").ayk_moe_route(
        _ptr(logits), c_int(logits.stride(0)), c_int(rows), c_int(logits.shape[1]), c_int(top),
        c_int(1 if over_all else 0), _ptr(chosen), _ptr(share), _stream())
    check(status, op)


def moe_experts(hidden: torch.Tensor, w_in: torch.Tensor, w_out: torch.Tensor,
                chosen: torch.Tensor, pair_out: torch.Tensor, *, experts: int, top: int,
                limit: float, alpha: float, sorted_pairs: torch.Tensor,
                tile_expert: torch.Tensor, inner: torch.Tensor, rows: int,
                shift: float = 1.0, single: bool = False) -> None:
    """The chosen experts of every row, as two products grouped by expert. ``w_in``
    ``[experts * 2 * ff, width]`` holds each expert's gate rows, then its up rows; ``w_out``
    ``[experts * width, ff]`` its down matrix. Pair ``p = row * top + choice`` computes
    ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + shift)`` and ``pair_out[p] = W_down y`` (float32
    ``[N * top, width]``, unweighted); ``limit=inf, alpha=1, shift=0`` is ``silu(g) * u``. Scratch: ``sorted_pairs`` (int32, ``tiles * tile
    rows``), ``tile_expert`` (int32, ``tiles``) and ``inner`` (``[tiles * tile rows, ff]``,
    compute dtype) sized by :func:`moe_scratch`. With ``single`` an expert has no gate:
    ``w_in`` is ``[experts * ff, width]`` and ``y = relu(W_up h)^2``."""
    op = "moe_experts"
    if _left_out and op in _left_out:
        return
    _need(op, "hidden", hidden, ndim=2)
    _need(op, "w_in", w_in, hidden.dtype, 2)
    _need(op, "w_out", w_out, hidden.dtype, 2)
    _need(op, "inner", inner, hidden.dtype, 2)
    _need(op, "chosen", chosen, torch.int32, 1)
    _need(op, "pair_out", pair_out, torch.float32, 2)
    _need(op, "sorted_pairs", sorted_pairs, torch.int32, 1)
    _need(op, "tile_expert", tile_expert, torch.int32, 1)
    width, ff = hidden.shape[1], w_out.shape[1]
    tile_rows = moe_tile_rows(rows, experts, top, hidden.dtype)
    tiles = moe_max_tiles(rows, experts, top, tile_rows)
    if hidden.dtype not in _TYPE or not w_in.is_contiguous() or not w_out.is_contiguous() or \
            tuple(w_in.shape) != (experts * (1 if single else 2) * ff, width) or \
            tuple(w_out.shape) != (experts * width, ff) or inner.shape[1] != ff or \
            pair_out.shape[1] != width or rows > hidden.shape[0] or \
            chosen.shape[0] < rows * top or pair_out.shape[0] < rows * top or \
            sorted_pairs.shape[0] < tiles * tile_rows or tile_expert.shape[0] < tiles or \
            inner.shape[0] < tiles * tile_rows:
        raise BackendError(f"{op}: shapes do not fit")
    global _launches
    _launches += 2  # align and two products
    status = library("moe").ayk_moe_experts(
        _ptr(hidden), c_int(hidden.stride(0)), _ptr(w_in), _ptr(w_out), _ptr(chosen),
        c_int(rows), c_int(experts), c_int(top), c_int(width), c_int(ff), c_float(limit),
        c_float(alpha), c_float(shift), c_int(1 if single else 0), _ptr(sorted_pairs),
        _ptr(tile_expert), c_int(tiles),
        c_int(tile_rows),
        _ptr(inner),
        c_int(inner.stride(0)), _ptr(pair_out), c_int(pair_out.stride(0)),
        c_int(_TYPE[hidden.dtype]), _stream())
    check(status, op)


def moe_join(pair_out: torch.Tensor, share: torch.Tensor, dst: torch.Tensor, *, top: int,
             scale: torch.Tensor | None = None, accumulate: bool = True, rows: int) -> None:
    """``dst[row] (+)= scale * sum_j share[row * top + j] * pair_out[row * top + j]`` in
    float32, the choices in order; ``scale`` (float32 ``[width]``) is optional."""
    op = "moe_join"
    if _left_out and op in _left_out:
        return
    _need(op, "pair_out", pair_out, torch.float32, 2)
    _need(op, "share", share, torch.float32, 1)
    _need(op, "dst", dst, torch.float32, 2)
    width = dst.shape[1]
    if pair_out.shape[1] != width or pair_out.shape[0] < rows * top or \
            share.shape[0] < rows * top or rows > dst.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    if scale is not None:
        _need(op, "scale", scale, torch.float32, 1)
        if scale.shape[0] != width:
            raise BackendError(f"{op}: the scale does not match the width")
    status = library("moe").ayk_moe_join(
        _ptr(pair_out), c_int(pair_out.stride(0)), _ptr(share), c_int(rows), c_int(top),
        _ptr(scale), _ptr(dst), c_int(dst.stride(0)), c_int(width),
        c_int(1 if accumulate else 0), _stream())
    check(status, op)


def moe_route_scored(logits: torch.Tensor, chosen: torch.Tensor, share: torch.Tensor, *,
                     top: int, groups: int = 1, keep: int = 1, factor: float = 1.0,
                     renormalise: bool = False, rows: int) -> None:
    """Routing by scores ``s = sigmoid(logits)`` (float32 ``[N, experts]``): the experts form
    ``groups`` equal groups of neighbours, a group's score is the sum of its two largest ``s``,
    only experts of the ``keep`` best groups can be chosen, and of those the ``top`` largest
    are (ties to the smaller index), in descending order, into ``chosen`` (int32 ``[N * top]``).
    ``share`` (float32 ``[N * top]``) gets ``factor * s``, divided by the chosen ones' sum
    with ``renormalise``."""
    op = "moe_route_scored"
    if _left_out and op in _left_out:
        return
    _need(op, "logits", logits, torch.float32, 2)
    _need(op, "chosen", chosen, torch.int32, 1)
    _need(op, "share", share, torch.float32, 1)
    if rows > logits.shape[0] or min(chosen.shape[0], share.shape[0]) < rows * top:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("moe").ayk_moe_route_scored(
        _ptr(logits), c_int(logits.stride(0)), c_int(rows), c_int(logits.shape[1]), c_int(top),
        c_int(groups), c_int(keep), c_float(factor), c_int(1 if renormalise else 0),
        _ptr(chosen), _ptr(share), _stream())
    check(status, op)


# ---- sublayers that read the residual stream itself, gated units ----------------------------

GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def cast_rows(x: torch.Tensor, out: torch.Tensor, *, rows: int) -> None:
    """``out = x`` (float32 ``[N, width]``) in ``out``'s type (float32 or bfloat16)."""
    op = "cast_rows"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "out", out, ndim=2)
    if out.dtype not in _TYPE or out.shape[1] != x.shape[1] or rows > x.shape[0] or \
            rows > out.shape[0]:
        raise BackendError(f"{op}: shapes or types do not fit")
    status = library("gated").ayk_cast_rows(
        _ptr(x), c_int(x.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(rows),
        c_int(x.shape[1]), c_int(_TYPE[out.dtype]), _stream())
    check(status, op)


def gated_unit(gate: torch.Tensor, out: torch.Tensor, *, activation: str, rows: int,
               other: torch.Tensor | None = None, table: torch.Tensor | None = None,
               index: torch.Tensor | None = None, column: int = 0) -> None:
    """``out = act(gate) * other`` entry by entry in fp32 (``act``: ``silu`` or ``gelu_tanh``;
    ``gate`` and ``other`` float32 ``[N, width]``), or, with ``table`` (``out``'s type) and
    ``index`` (int32 per row), ``out[r] = act(gate[r]) * table[index[r], column : column +
    width]``."""
    op = "gated_unit"
    if _left_out and op in _left_out:
        return
    _need(op, "gate", gate, torch.float32, 2)
    _need(op, "out", out, ndim=2)
    width = out.shape[1]
    if out.dtype not in _TYPE or activation not in GATE_ACTIVATIONS or gate.shape[1] != width \
            or rows > gate.shape[0] or rows > out.shape[0] or (other is None) == (table is None):
        raise BackendError(f"{op}: shapes, types or arguments do not fit")
    if other is not None:
        _need(op, "other", other, torch.float32, 2)
        if other.shape[1] != width or rows > other.shape[0]:
            raise BackendError(f"{op}: other does not match gate")
    else:
        _need(op, "table", table, out.dtype, 2)
        _need(op, "index", index, torch.int32, 1)
        if column < 0 or table.shape[1] < column + width or rows > index.shape[0]:
            raise BackendError(f"{op}: the table has no such columns")
    status = library("gated").ayk_gated_unit(
        _ptr(gate), c_int(gate.stride(0)), _ptr(other),
        c_int(0 if other is None else other.stride(0)), _ptr(table),
        c_int(0 if table is None else table.stride(0)), _ptr(index),
        c_int(0 if table is None else table.shape[0]), c_int(column),
        c_int(GATE_ACTIVATIONS[activation]), _ptr(out), c_int(out.stride(0)), c_int(rows),
        c_int(width), c_int(_TYPE[out.dtype]), _stream())
    check(status, op)


UNARY_ACTIVATIONS = {"tanh": 0, "xielu": 1}


def unary_rows(x: torch.Tensor, out: torch.Tensor, *, activation: str, rows: int,
               bias: torch.Tensor | None = None, numbers: torch.Tensor | None = None) -> None:
    """``out = act(x + bias)`` entry by entry in fp32 (``x`` float32 ``[N, width]``, ``out``
    float32 or bfloat16). ``act``: ``tanh``, or ``xielu`` with ``numbers`` = float32 ``(p, q)``:
    ``softplus(p) z^2 + z / 2`` for ``z > 0``, ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``
    otherwise."""
    op = "unary_rows"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "out", out, ndim=2)
    width = out.shape[1]
    if out.dtype not in _TYPE or activation not in UNARY_ACTIVATIONS or x.shape[1] != width \
            or rows > x.shape[0] or rows > out.shape[0]:
        raise BackendError(f"{op}: shapes, types or arguments do not fit")
    if bias is not None:
        _need(op, "bias", bias, torch.float32, 1)
        if bias.shape[0] != width:
            raise BackendError(f"{op}: the bias does not match the width")
    if activation == "xielu":
        _need(op, "numbers", numbers, torch.float32, 1)
        if numbers.shape[0] != 2:
            raise BackendError(f"{op}: xielu takes two numbers")
    status = library("gated").ayk_unary_rows(
        _ptr(x), c_int(x.stride(0)), _ptr(bias), c_int(UNARY_ACTIVATIONS[activation]),
        _ptr(numbers), _ptr(out), c_int(out.stride(0)), c_int(rows), c_int(width),
        c_int(_TYPE[out.dtype]), _stream())
    check(status, op)


def delta_scan(proj: torch.Tensor, decay: torch.Tensor, rate_bias: torch.Tensor,
               state: torch.Tensor, out: torch.Tensor, *, row_start: torch.Tensor,
               state_slot: torch.Tensor, requests: int, heads: int, dim: int, columns: int,
               k_offset: int, v_offset: int, a_offset: int, decay_rate: float) -> None:
    """The generalised delta rule over the step's rows, request by request, from and into each
    request's slot of ``state`` (float32 ``[slots, heads * columns * dim]``, ``S`` kept as
    ``[head][column][key channel]``). ``proj`` (float32) holds per row the receptance at column
    0, the key at ``k_offset``, the raw removal rate at ``a_offset`` (``heads x dim`` each) and
    the value at ``v_offset`` (``heads x columns``); ``decay`` (float32 ``[N, heads * dim]``)
    the raw decays. Per head, with ``u = k / sqrt(k . k + 1e-6)``,
    ``w = exp(-decay_rate * sigmoid(decay))`` and ``a = sigmoid(rate + rate_bias)``:
    ``S <- diag(w) S - (a * u)(u^T S) + k v^T`` (both terms from the old ``S``) and
    ``out = S^T r`` (float32 ``[N, heads * columns]``)."""
    op = "delta_scan"
    if _left_out and op in _left_out:
        return
    _need(op, "proj", proj, torch.float32, 2)
    _need(op, "decay", decay, torch.float32, 2)
    _need(op, "rate_bias", rate_bias, torch.float32, 1)
    _need(op, "state", state, torch.float32, 2)
    _need(op, "out", out, torch.float32, 2)
    _need(op, "row_start", row_start, torch.int32, 1)
    _need(op, "state_slot", state_slot, torch.int32, 1)
    if rate_bias.shape[0] != heads * dim or decay.shape[1] < heads * dim or \
            out.shape[1] < heads * columns or state.shape[1] < heads * dim * columns or \
            row_start.shape[0] < requests + 1 or state_slot.shape[0] < requests:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("recurrent").ayk_delta_scan(
        _ptr(proj), c_int(proj.stride(0)), c_int(k_offset), c_int(v_offset), c_int(a_offset),
        _ptr(rate_bias), _ptr(decay), c_int(decay.stride(0)), c_float(decay_rate), _ptr(state),
        c_longlong(state.stride(0)), _ptr(row_start), _ptr(state_slot), _ptr(out),
        c_int(out.stride(0)), c_int(requests), c_int(heads), c_int(dim), c_int(columns),
        _stream())
    check(status, op)


def pooled_prepare(proj: torch.Tensor, *, k_offset: int, q_weight: torch.Tensor | None,
                   k_weight: torch.Tensor | None, eps: float, positions: torch.Tensor,
                   freq: torch.Tensor | None, rot_dims: int, rot_gain: float,
                   slot_mapping: torch.Tensor | None, k_pages: torch.Tensor | None,
                   v_pages: torch.Tensor | None, q: torch.Tensor, heads: int, kv_heads: int,
                   dim: int, rows: int) -> None:
    """From a row of the fused projection (float32: queries at column 0, keys at
    ``k_offset``): every head divided by its own root mean square and multiplied by one weight
    of ``dim`` entries shared by the heads (``q_weight`` / ``k_weight``; ``None``: no norm),
    the first ``rot_dims`` entries of each head rotated by the row's position (entry ``i`` with
    ``i + rot_dims / 2``, cosine and sine times ``rot_gain``); queries into ``q``, keys into the
    row's slot of ``k_pages`` and the *raw* key rows (before norm and rotation) into
    ``v_pages`` as the token's value."""
    op = "pooled_prepare"
    if _left_out and op in _left_out:
        return
    _need(op, "proj", proj, torch.float32, 2)
    _need(op, "q", q, ndim=2)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or rows > proj.shape[0] or rows > q.shape[0] or \
            rows > positions.shape[0] or q.shape[1] != heads * dim or \
            proj.shape[1] < k_offset + kv_heads * dim:
        raise BackendError(f"{op}: shapes do not fit")
    page_size = 0
    if k_pages is not None:
        _need(op, "k_pages", k_pages, q.dtype, 4)
        _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
        if not k_pages.is_contiguous() or tuple(k_pages.shape[1:]) != \
                (kv_heads, k_pages.shape[2], dim) or rows > slot_mapping.shape[0]:
            raise BackendError(f"{op}: the key pages do not fit")
        page_size = k_pages.shape[2]
        if v_pages is not None:
            _need(op, "v_pages", v_pages, q.dtype, 4)
            if not v_pages.is_contiguous() or tuple(v_pages.shape) != tuple(k_pages.shape):
                raise BackendError(f"{op}: raw keys as values need value pages like the key "
                                   "pages")
    if rot_dims:
        _need(op, "freq", freq, torch.float64, 1)
        if freq.shape[0] != rot_dims // 2:
            raise BackendError(f"{op}: one frequency per rotated pair")
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _need(op, name, weight, torch.float32, 1)
            if weight.shape[0] != dim:
                raise BackendError(f"{op}: the norm weights have one entry per head entry")
    status = library("pooled_attention").ayk_pooled_prepare(
        _ptr(proj), c_int(proj.stride(0)), c_int(k_offset), _ptr(q_weight), _ptr(k_weight),
        c_float(eps), _ptr(positions), _ptr(freq), c_int(rot_dims), c_float(rot_gain),
        _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages), c_int(page_size), _ptr(q),
        c_int(q.stride(0)), c_int(rows), c_int(heads), c_int(kv_heads), c_int(dim),
        c_int(_TYPE[q.dtype]), _stream())
    check(status, op)


def pool_slots(page_size: int, pool: int) -> int:
    """Pooled rows a page of ``page_size`` tokens holds for blocks of ``pool`` tokens."""
    return -(-page_size // pool)


def pooled_blocks(k_pages: torch.Tensor, v_pages: torch.Tensor, k_pool: torch.Tensor,
                  v_pool: torch.Tensor, block_table: torch.Tensor, request_of_row: torch.Tensor,
                  positions: torch.Tensor, row_start: torch.Tensor, *, pool: int, rows: int,
                  requests: int) -> None:
    """For every block of ``pool`` positions whose last position is among the step's rows
    (request ``b`` brings the rows ``row_start[b] .. row_start[b + 1]`` at consecutive
    positions): the mean of the block's cached keys into ``k_pool`` and of its cached values
    into ``v_pool`` (``[pages, kv_heads, pool_slots, dim]``), in the page of the block's first
    position, at slot ``(first % page_size) // pool``."""
    op = "pooled_blocks"
    if _left_out and op in _left_out:
        return
    _need(op, "k_pages", k_pages, ndim=4)
    _need(op, "v_pages", v_pages, k_pages.dtype, 4)
    _need(op, "k_pool", k_pool, k_pages.dtype, 4)
    _need(op, "v_pool", v_pool, k_pages.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    _need(op, "row_start", row_start, torch.int32, 1)
    pages, kv_heads, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    slots = pool_slots(page_size, pool) if pool > 0 else 0
    if k_pages.dtype not in _TYPE or pool < 1 or \
            tuple(k_pool.shape) != (pages, kv_heads, slots, dim) or \
            tuple(v_pool.shape) != (pages, kv_heads, slots, vdim) or \
            not all(t.is_contiguous() for t in (k_pages, v_pages, k_pool, v_pool)) or \
            rows > positions.shape[0] or rows > request_of_row.shape[0] or \
            row_start.shape[0] < requests + 1 or block_table.shape[0] < requests:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("pooled_attention").ayk_pooled_blocks(
        _ptr(positions), _ptr(request_of_row), _ptr(row_start), c_int(requests),
        _ptr(block_table), c_int(block_table.stride(0)),
        _ptr(k_pages), _ptr(v_pages), _ptr(k_pool), _ptr(v_pool), c_int(page_size), c_int(pool),
        c_int(slots), c_int(rows), c_int(kv_heads), c_int(dim), c_int(vdim),
        c_int(_TYPE[k_pages.dtype]), _stream())
    check(status, op)


def pooled_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
                     block_table: torch.Tensor, request_of_row: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, *, heads: int, scale: float,
                     window: int, pool: int, sink: torch.Tensor | None, rows: int,
                     shares: int = 0, partial: torch.Tensor | None = None) -> bool:
    """Softmax attention of ``rows`` rows over the paged cache: the row at position ``p`` sees
    the keys ``j`` with ``0 <= p - j < window`` (``window`` 0: all earlier keys) and, with
    ``pool`` > 0, the pooled rows of the blocks ``e < (p - window + 1) // pool``; the
    denominator also holds ``exp(sink[head])`` when ``sink`` (float32 ``[heads]``) is given.
    ``shares`` 0: one CTA per (row, head), any sizes; ``shares`` >= 1: a row's entries cut into
    that many shares (``partial``: float32 scratch of ``rows * heads * shares * (vdim + 2)``
    elements when more than one). Returns False, having run nothing, when the kernel of
    shares does not take the sizes."""
    global _launches
    op = "pooled_attention"
    if _left_out and op in _left_out:
        return True
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    pages, kv_heads, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    if q.shape[1] != heads * dim or out.shape[1] != heads * vdim or \
            tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3]) or rows > out.shape[0] or \
            rows > q.shape[0] or rows > request_of_row.shape[0] or \
            rows > positions.shape[0] or heads % kv_heads or shares < 0:
        raise BackendError(f"{op}: shapes do not fit")
    slots = 0
    if pool > 0 and window > 0:
        slots = pool_slots(page_size, pool)
        _need(op, "k_pool", k_pool, q.dtype, 4)
        _need(op, "v_pool", v_pool, q.dtype, 4)
        if tuple(k_pool.shape) != (pages, kv_heads, slots, dim) or \
                tuple(v_pool.shape) != (pages, kv_heads, slots, vdim) or \
                not k_pool.is_contiguous() or not v_pool.is_contiguous():
            raise BackendError(f"{op}: the pooled rows do not match the pages")
    if sink is not None:
        _need(op, "sink", sink, torch.float32, 1)
        if sink.shape[0] != heads:
            raise BackendError(f"{op}: one sink per head")
    if shares > 1:
        if partial is None:
            raise BackendError(f"{op}: more than one share needs scratch")
        _need(op, "partial", partial, torch.float32)
        if partial.numel() < rows * heads * shares * (vdim + 2):
            raise BackendError(f"{op}: the scratch is too small")
    status = library("pooled_attention").ayk_pooled_attention(
        _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions),
        _ptr(sink), _ptr(partial if shares > 1 else None), _ptr(out), c_int(out.stride(0)),
        c_int(rows), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(page_size),
        c_float(scale), c_int(window), c_int(pool), c_int(slots), c_int(shares),
        c_int(_TYPE[q.dtype]), _stream())
    if status == -6:  # the kernel of shares does not take these sizes
        return False
    check(status, op)
    if shares > 1:
        _launches += 1  # the merge
    return True


def norm_add(x: torch.Tensor, weight: torch.Tensor, eps: float, dst: torch.Tensor, *,
             factor: float = 1.0, weight_offset: float = 0.0, copy: torch.Tensor | None = None,
             rows: int, next_weight: torch.Tensor | None = None, next_eps: float = 1e-6,
             next_offset: float = 0.0, next_out: torch.Tensor | None = None) -> None:
    """``dst += factor * x * rsqrt(mean(x^2) + eps) * (weight_offset + weight)`` over float32
    rows; with ``copy`` (float32 or bfloat16 ``[N, width]``) the new ``dst`` is also written
    there, rounded once; with ``next_out`` (of ``copy``'s type when both are given) and
    ``next_weight`` the new ``dst`` also leaves normalised for the sublayer that follows:
    ``next_out = dst * rsqrt(mean(dst^2) + next_eps) * (next_offset + next_weight)``."""
    op = "norm_add"
    if _left_out and op in _left_out:
        return
    _need(op, "x", x, torch.float32, 2)
    _need(op, "weight", weight, torch.float32, 1)
    _need(op, "dst", dst, torch.float32, 2)
    width = dst.shape[1]
    if x.shape[1] != width or weight.shape[0] != width or rows > x.shape[0] or \
            rows > dst.shape[0]:
        raise BackendError(f"{op}: shapes do not fit")
    if copy is not None:
        _need(op, "copy", copy, ndim=2)
        if copy.dtype not in _TYPE or copy.shape[1] != width or rows > copy.shape[0]:
            raise BackendError(f"{op}: the copy does not match dst")
    typed = copy
    if next_out is not None:
        _need(op, "next_out", next_out, ndim=2)
        _need(op, "next_weight", next_weight, torch.float32, 1)
        if next_out.dtype not in _TYPE or next_out.shape[1] != width or \
                rows > next_out.shape[0] or next_weight.shape[0] != width or \
                (copy is not None and copy.dtype != next_out.dtype):
            raise BackendError(f"{op}: the next norm's output does not match dst")
        typed = next_out
    status = library("rms_norm").ayk_norm_add_next(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), c_float(weight_offset), c_float(eps),
        c_float(factor), _ptr(dst), c_int(dst.stride(0)), _ptr(copy),
        c_int(0 if copy is None else copy.stride(0)),
        c_int(0 if typed is None else _TYPE[typed.dtype]),
        _ptr(next_weight if next_out is not None else None), c_float(next_offset),
        c_float(next_eps), _ptr(next_out),
        c_int(0 if next_out is None else next_out.stride(0)), c_int(rows), c_int(width),
        _stream())
    check(status, op)


# ---- attention with a window that keeps the first tokens, and an output gate ----------------

def gated_attention_prepare(proj: torch.Tensor, *, k_offset: int, v_offset: int,
                            q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                            eps: float, slot_mapping: torch.Tensor | None,
                            k_pages: torch.Tensor | None, v_pages: torch.Tensor | None,
                            q: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                            rows: int) -> None:
    """From a row of a fused projection (float32: ``heads * dim`` queries at 0, ``kv_heads *
    dim`` keys at ``k_offset``, ``kv_heads * vdim`` values at ``v_offset``): queries and keys
    each normalised by the root mean square over their whole projection with a weight per
    entry (``None``: no norm), the queries written to ``q`` ``[N, heads * dim]``, the key and
    value into the row's cache slot (``k_pages`` ``[page, kv_head, slot, dim]``, ``v_pages``
    likewise with ``vdim``; ``None``: stored nowhere)."""
    op = "gated_attention_prepare"
    if _left_out and op in _left_out:
        return
    _need(op, "proj", proj, torch.float32, 2)
    _need(op, "q", q, ndim=2)
    if q.dtype not in _TYPE:
        raise BackendError(f"{op}: float32 or bfloat16 only")
    for name, tensor, size in (("q_weight", q_weight, heads * dim),
                               ("k_weight", k_weight, kv_heads * dim)):
        if tensor is not None:
            _need(op, name, tensor, torch.float32)
            if tensor.numel() != size or not tensor.is_contiguous():
                raise BackendError(f"{op}: {name} must hold {size} contiguous entries")
    page_size = 1
    if k_pages is not None:
        if v_pages is None or slot_mapping is None:
            raise BackendError(f"{op}: key pages come with value pages and a slot mapping")
        _need(op, "k_pages", k_pages, q.dtype, 4)
        _need(op, "v_pages", v_pages, q.dtype, 4)
        _need(op, "slot_mapping", slot_mapping, torch.int32, 1)
        page_size = k_pages.shape[2]
        if tuple(k_pages.shape[1:]) != (kv_heads, page_size, dim) or \
                tuple(v_pages.shape[1:]) != (kv_heads, page_size, vdim) or \
                not k_pages.is_contiguous() or not v_pages.is_contiguous() or \
                rows > slot_mapping.shape[0]:
            raise BackendError(f"{op}: pages must be contiguous [page, kv_head, slot, dim]")
    if rows > proj.shape[0] or rows > q.shape[0] or q.shape[1] != heads * dim or \
            proj.shape[1] < v_offset + kv_heads * vdim:
        raise BackendError(f"{op}: shapes do not fit")
    status = library("gated_attention").ayk_gated_prepare(
        _ptr(proj), c_int(proj.stride(0)), c_int(k_offset), c_int(v_offset), _ptr(q_weight),
        _ptr(k_weight), c_float(eps), _ptr(slot_mapping if k_pages is not None else None),
        _ptr(k_pages), _ptr(v_pages), c_int(page_size), _ptr(q), c_int(q.stride(0)),
        c_int(rows), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim),
        c_int(_TYPE[q.dtype]), _stream())
    check(status, op)


def gated_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    block_table: torch.Tensor, request_of_row: torch.Tensor,
                    positions: torch.Tensor, out: torch.Tensor, *, heads: int, scale: float,
                    window: int = 0, keep_first: int = 0, gate: torch.Tensor | None = None,
                    rows: int | None = None, tensor_cores: bool = True) -> None:
    """Softmax attention over paged keys (``[page, kv_head, slot, dim]``) and values (``[...,
    vdim]``): the row of request ``request_of_row[i]`` at ``positions[i]`` sees key ``j <= p``
    when ``p - j < window`` (``window`` 0: always) or ``j < keep_first``; head ``h`` uses
    key/value head ``h // (heads / kv_heads)``; scores ``scale * q . k`` and the softmax in
    fp32; with ``gate`` (float32 ``[N, heads * vdim]``) the result is multiplied entry by
    entry by ``sigmoid(gate)``. The step's own keys must already be stored."""
    op = "gated_attention"
    if _left_out and op in _left_out:
        return
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    n = q.shape[0] if rows is None else rows
    if q.shape[1] != heads * dim or out.shape[1] != heads * vdim or \
            tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3]) or n > out.shape[0] or \
            n > request_of_row.shape[0] or n > positions.shape[0] or heads % kv_heads:
        raise BackendError(f"{op}: shapes do not fit")
    if gate is not None:
        _need(op, "gate", gate, torch.float32, 2)
        if gate.shape[1] != heads * vdim or gate.shape[0] < n:
            raise BackendError(f"{op}: the gate does not match the rows")
    status = library("gated_attention").ayk_gated_attention(
        _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(gate),
        c_int(0 if gate is None else gate.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(n),
        c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(page_size),
        c_float(scale), c_int(window), c_int(keep_first), c_int(1 if tensor_cores else 0),
        c_int(_TYPE[q.dtype]), _stream())
    check(status, op)


def gated_decode_shares(rows: int, heads: int, reach: int,
                        device: torch.device | None = None) -> int:
    """Shares a row's visible keys are cut into by :func:`gated_decode`: down to one tile of
    128 keys a share while that gives no more than eight CTAs per SM over all rows and heads;
    at most 32."""
    want = -(-8 * sm_count(device) // max(1, rows * heads))
    return max(1, min(want, -(-reach // 128), 32))


def gated_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 block_table: torch.Tensor, request_of_row: torch.Tensor,
                 positions: torch.Tensor, out: torch.Tensor, partial: torch.Tensor | None, *,
                 heads: int, scale: float, window: int = 0, keep_first: int = 0,
                 gate: torch.Tensor | None = None, rows: int, shares: int) -> bool:
    """:func:`gated_attention` for steps of single rows: a row's visible keys are cut into
    ``shares`` shares, one CTA each per head, and joined in their order. ``partial`` is
    float32 scratch of at least ``rows * heads * shares * (vdim + 2)`` elements (``None`` with
    one share). Returns False, having run nothing, for sizes the kernel does not take (value
    rows that are not whole 16-byte pieces)."""
    op = "gated_decode"
    if _left_out and ("gated_attention" in _left_out or op in _left_out):
        return True
    _need(op, "q", q, ndim=2)
    _need(op, "out", out, q.dtype, 2)
    _need(op, "k_pages", k_pages, q.dtype, 4)
    _need(op, "v_pages", v_pages, q.dtype, 4)
    _need(op, "block_table", block_table, torch.int32, 2)
    _need(op, "request_of_row", request_of_row, torch.int32, 1)
    _need(op, "positions", positions, torch.int32, 1)
    if q.dtype not in _TYPE or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise BackendError(f"{op}: contiguous float32 or bfloat16 pages only")
    _, kv_heads, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    if q.shape[1] != heads * dim or out.shape[1] != heads * vdim or \
            tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3]) or rows > out.shape[0] or \
            rows > q.shape[0] or rows > request_of_row.shape[0] or \
            rows > positions.shape[0] or heads % kv_heads or shares < 1:
        raise BackendError(f"{op}: shapes do not fit")
    if shares > 1:
        if partial is None:
            raise BackendError(f"{op}: more than one share needs scratch")
        _need(op, "partial", partial, torch.float32)
        if not partial.is_contiguous() or \
                partial.numel() < rows * heads * shares * (vdim + 2):
            raise BackendError(f"{op}: the scratch is too small")
    if gate is not None:
        _need(op, "gate", gate, torch.float32, 2)
        if gate.shape[1] != heads * vdim or gate.shape[0] < rows or gate.stride(1) != 1:
            raise BackendError(f"{op}: the gate does not match the rows")
    global _launches
    status = library("gated_attention").ayk_gated_decode(
        _ptr(q), c_int(q.stride(0)), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(request_of_row), _ptr(positions), _ptr(gate),
        c_int(0 if gate is None else gate.stride(0)), _ptr(partial if shares > 1 else None),
        _ptr(out), c_int(out.stride(0)), c_int(rows), c_int(heads), c_int(kv_heads),
        c_int(dim), c_int(vdim), c_int(page_size), c_float(scale), c_int(window),
        c_int(keep_first), c_int(shares), c_int(_TYPE[q.dtype]), _stream())
    if status == -6:  # AYK_NOT_TAKEN
        _launches -= 1
        return False
    if shares > 1:
        _launches += 1  # the merge of the shares is a launch of its own
    check(status, op)
    return True
