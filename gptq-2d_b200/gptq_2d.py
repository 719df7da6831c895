"""GPTQ-2D on B200: the public entry points of the reference's ``gptq_2d.py`` over hand-written sm_100a CUDA.

``gptq_2d``, ``gptq_2d_super_entry`` and ``capture_gptq_2d`` keep the reference's signatures and semantics
(gptq_2d.py:1379-1564 of IST-DASLab/GPTQ-2D): leading batch dimensions broadcast without copying L and U,
``inplace=True`` returns the caller's tensor, empty inputs return at once, nothing synchronizes with the host,
so every call can be captured in a CUDA graph.  Two engines sit behind them:

* the **fused engine** (``g2d_sweep_fused``) runs when the quantizer is one this package knows
  (``round_quantizer`` and the affine quantizers of ``quantizer_int``, also inside ``functools.partial``)
  and the entries are plain.  The quantizer is evaluated inside the sweep kernels, and the sweep is ordered
  by tiles instead of global antidiagonals -- any order in which an entry is rounded after everything above
  it and to its left gives the same result in exact arithmetic;
* the **generic engine** calls an arbitrary Python quantizer once per (coarse) antidiagonal, exactly as the
  reference does, with live Y, and pushes / flushes with the CUDA kernels ``g2d_stage_push`` / ``g2d_stage_flush``.

There is no Triton, no CPU path and no fallback: CPU tensors are rejected, and a missing CUDA library raises.
"""
from __future__ import annotations

import ctypes
import functools
from collections.abc import Callable

import torch

import _abi
import quantizer_int
from quantizer_int import round_quantizer, round_quantizer_super_entry

_Selection = slice | Callable[[torch.Tensor], torch.Tensor]


# --------------------------------------------------------------------------------------------------------
# validation and geometry (same contract and messages as gptq_2d.py:65-184 of the reference)
# --------------------------------------------------------------------------------------------------------

def _validate_inputs(x, l, u, inplace: bool, require_cuda: bool = True, super_entry_shape=(1, 1)):
    assert x.dim() >= 2 and l.dim() >= 2 and u.dim() >= 2, "X, L, and U must have at least two dimensions"
    m, n = x.shape[-2:]
    assert l.shape[-2:] == (m, m) and u.shape[-2:] == (n, n), "expected X=[...,m,n], L=[...,m,m], and U=[...,n,n]"
    p, q = super_entry_shape
    assert p > 0 and q > 0 and m % p == 0 and n % q == 0, "the super-entry shape must divide the matrix shape"
    assert x.dtype in (torch.float32, torch.float64) and x.dtype == l.dtype == u.dtype, "X, L, and U must share dtype float32 or float64"
    assert x.device == l.device == u.device, "X, L, and U must be on the same device"
    assert not require_cuda or x.is_cuda, "X, L, and U must be CUDA tensors"
    batch_shape = torch.broadcast_shapes(x.shape[:-2], l.shape[:-2], u.shape[:-2])
    assert not inplace or (x.is_contiguous() and x.shape[:-2] == batch_shape), "inplace=True requires contiguous X with the exact broadcast batch shape"
    return m, n, batch_shape


def _prepare_output(x, l, u, inplace, super_entry_shape=(1, 1)):
    m, n, batch_shape = _validate_inputs(x, l, u, inplace, True, super_entry_shape)
    y = x if inplace else x.expand(*batch_shape, m, n).clone(memory_format=torch.contiguous_format)
    return y, m, n, batch_shape


def _antidiagonal_slices(*, m: int, n: int, s: int, super_entry_shape=(1, 1)) -> tuple[slice, slice, slice]:
    """Coarse row slice, coarse column slice and the flat slice of the first entries of the super-entries of stage s.

    Super-entry (ibar, jbar) of a row-major matrix starts at flat position ``ibar*p*n + jbar*q``; along a coarse
    antidiagonal consecutive starts lie ``p*n - q`` apart (one super-entry's span when a stage holds a single one).
    """
    p, q = super_entry_shape
    first_row, end_row = max(0, s - n // q + 1), min(s + 1, m // p)
    step = max(p * n - q, (p - 1) * n + q)
    start = first_row * p * n + (s - first_row) * q
    return slice(first_row, end_row), slice(s - end_row + 1, s - first_row + 1), slice(start, start + (end_row - first_row) * step, step)


def _super_entries(x_flat: torch.Tensor, antidiagonal_slice: slice, n: int, super_entry_shape) -> torch.Tensor:
    """View ``[..., m*n]`` as the ``[..., d, p, q]`` super-entries of one coarse antidiagonal (writes go through)."""
    p, q = super_entry_shape
    window = x_flat[..., antidiagonal_slice.start:antidiagonal_slice.stop]
    return window.unfold(-1, (p - 1) * n + q, antidiagonal_slice.step).unfold(-1, q, n)


def _row_major(t: torch.Tensor) -> torch.Tensor:
    """A tensor whose matrices are dense row-major; broadcast (stride-0) batch dimensions are kept as they are."""
    k = t.size(-1)
    if t.stride(-1) == 1 and t.stride(-2) == k or t.numel() == 0:
        return t
    return t.contiguous()


# --------------------------------------------------------------------------------------------------------
# fused engine
# --------------------------------------------------------------------------------------------------------

# Launch schedule of the fused engine: 0 lets the library choose, 1 forces the tile schedule (64 x 64 tiles, FFMA
# updates), 2 forces the macro schedule (128 x 128 macro tiles; tensor-core updates where the library has them),
# 3 the pipelined schedule (tile launches on the critical path only, tensor-core updates on side streams; float32).
SWEEP_SCHEDULE = 0

_AFFINE_PLAIN = (quantizer_int.affine_quantizer_cuda,)
_AFFINE_SUPER = (quantizer_int.affine_quantizer_super_entry_cuda,)


def _fusable(quantizer: Callable, quantizer_inputs, super_entry_shape) -> dict | None:
    """Recognise a quantizer of this package and return the options of the engine that has it inside its kernels, or
    None.  Plain entries (and 1 x 1 super-entries) under the round and affine quantizers go to the fused tile engine;
    larger super-entries, the dynamic abs-max quantizer and the trellis quantizer to the library's super-entry sweep
    (``super=True`` in the options), whose whole stage loop runs inside one C call."""
    import quantizer_trellis

    func, keywords = quantizer, {}
    while isinstance(func, functools.partial):
        if func.args:
            return None
        keywords = {**func.keywords, **keywords}
        func = func.func
    plain = super_entry_shape is None
    single = plain or tuple(super_entry_shape) == (1, 1)
    if func is (round_quantizer if plain else round_quantizer_super_entry) and not keywords and not quantizer_inputs:
        return dict(kind=_abi.Q_ROUND, super=not single)
    if func in (_AFFINE_PLAIN if plain else _AFFINE_SUPER) and len(quantizer_inputs) == 2 and set(keywords) <= {"qmin", "qmax"}:
        return dict(kind=_abi.Q_AFFINE, qmin=keywords.get("qmin", -torch.inf), qmax=keywords.get("qmax", torch.inf), super=not single)
    if plain:
        return None
    if func is quantizer_int.int_abs_max_quantizer_cuda and not quantizer_inputs and set(keywords) == {"qmin", "qmax", "dtype"}:
        if keywords["dtype"] in (torch.float16, torch.bfloat16) and keywords["qmin"] < keywords["qmax"]:
            return dict(kind=_abi.Q_ABSMAX_DYNAMIC, qmin=keywords["qmin"], qmax=keywords["qmax"], half=_abi.half_code(keywords["dtype"]), super=True)
    if (func is quantizer_trellis.trellis_quantizer_super_entry_cuda and len(quantizer_inputs) == 1
            and {"table", "K"} <= set(keywords) <= {"table", "K", "tail_biting"}):
        table, K, (p, q) = keywords["table"], keywords["K"], super_entry_shape
        if table.dim() == 2 and table.size(1) <= 2 and K * table.size(1) <= 8 and (p * q) % table.size(1) == 0 and table.size(0) & (table.size(0) - 1) == 0:
            return dict(kind=_abi.Q_TRELLIS, table=table, K=K, tail_biting=keywords.get("tail_biting", True), super=True)
    return None


def _matrix_strides(t: torch.Tensor, m: int, n: int) -> tuple[int, int]:
    return (t.stride(-2) if m > 1 else 0), (t.stride(-1) if n > 1 else 0)


def _sweep_fused(y, l, u, batch_shape, options: dict, quantizer_inputs, *, forced_z=None, y_pre=None, outer_tiles: int = 0):
    m, n = y.shape[-2:]
    lib = _abi.library()
    l, u = _row_major(l), _row_major(u)
    desc = _abi.SweepDesc()
    desc.dtype, desc.quant_kind = _abi.dtype_code(y.dtype), options["kind"]
    desc.batch, desc.m, desc.n = batch_shape.numel(), m, n
    keep = [l, u, _abi.batch_offsets(l, batch_shape), _abi.batch_offsets(u, batch_shape)]
    desc.y, desc.l, desc.u = y.data_ptr(), l.data_ptr(), u.data_ptr()
    desc.l_offsets, desc.u_offsets = _abi.ptr(keep[2]), _abi.ptr(keep[3])
    if options["kind"] == _abi.Q_AFFINE:
        scale, zero = quantizer_inputs
        y_flat = y.flatten(start_dim=-2)
        out_like = y_flat  # only shapes, dtype and device are checked
        quantizer_int._validate_affine_inputs(y_flat, scale, zero, out_like, options["qmin"], options["qmax"])
        assert scale.shape[-2:] == (m, n), "scale and zero point matrix shapes must match Y"
        so, zo = _abi.batch_offsets(scale, batch_shape), _abi.batch_offsets(zero, batch_shape)
        keep += [scale, zero, so, zo]
        desc.scale, desc.zero, desc.scale_offsets, desc.zero_offsets = scale.data_ptr(), zero.data_ptr(), _abi.ptr(so), _abi.ptr(zo)
        desc.scale_row_stride, desc.scale_col_stride = _matrix_strides(scale, m, n)
        desc.zero_row_stride, desc.zero_col_stride = _matrix_strides(zero, m, n)
        desc.qmin, desc.qmax = float(options["qmin"]), float(options["qmax"])
    if forced_z is not None:
        desc.forced_z = forced_z.data_ptr()
    if y_pre is not None:
        desc.y_pre = y_pre.data_ptr()
    desc.outer_tiles = outer_tiles
    desc.reserved = SWEEP_SCHEDULE
    desc.status = _abi.status_word(y.device).data_ptr()
    size = ctypes.c_size_t()
    _abi.check(lib.g2d_sweep_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)), "g2d_sweep_workspace_bytes")
    workspace = torch.empty(size.value, dtype=torch.uint8, device=y.device)
    desc.workspace, desc.workspace_bytes = workspace.data_ptr(), size.value
    with torch.cuda.device(y.device):
        _abi.check(lib.g2d_sweep_fused(ctypes.byref(desc), _abi.stream_of(y)), "g2d_sweep_fused")
    return y


def _sweep_super(y, l, u, batch_shape, options: dict, quantizer_inputs, super_entry_shape, inner_block_size, outer_block_size, *,
                 lead_factors=(), codes: torch.Tensor | None = None):
    """The library's super-entry sweep (``g2d_sweep_super_entry``): the stage loop, the quantizer and the pushes in one C
    call.  ``lead_factors``: the leading modes' factors of an N-factor sweep, y then being ``[*lead sizes, m, n]``.
    Returns None when the inputs have a form the library does not take (the caller then uses the per-stage engine)."""
    m, n = y.shape[-2:]
    p, q = super_entry_shape or (1, 1)
    lib = _abi.library()
    l, u = _row_major(l), _row_major(u)
    desc = _abi.SuperDesc()
    desc.dtype, desc.quant_kind, desc.p, desc.q = _abi.dtype_code(y.dtype), options["kind"], p, q
    desc.inner_block, desc.outer_block = inner_block_size, outer_block_size
    desc.batch, desc.m, desc.n = batch_shape.numel(), m, n
    keep = [l, u, _abi.batch_offsets(l, batch_shape), _abi.batch_offsets(u, batch_shape)]
    desc.y, desc.l, desc.u = y.data_ptr(), l.data_ptr(), u.data_ptr()
    desc.l_offsets, desc.u_offsets = _abi.ptr(keep[2]), _abi.ptr(keep[3])
    desc.lead_count = len(lead_factors)
    for k, factor in enumerate(lead_factors):
        factor = factor.contiguous()
        keep.append(factor)
        desc.lead_size[k], desc.lead_factor[k] = factor.size(0), factor.data_ptr()
    kind = options["kind"]
    if kind == _abi.Q_AFFINE:
        scale, zero = quantizer_inputs
        y_flat = y.flatten(start_dim=-2)
        quantizer_int._validate_affine_inputs(y_flat, scale, zero, y_flat, options["qmin"], options["qmax"])
        so, zo = _abi.batch_offsets(scale, batch_shape), _abi.batch_offsets(zero, batch_shape)
        keep += [scale, zero, so, zo]
        desc.scale, desc.zero, desc.scale_offsets, desc.zero_offsets = scale.data_ptr(), zero.data_ptr(), _abi.ptr(so), _abi.ptr(zo)
        desc.scale_row_stride, desc.scale_col_stride = _matrix_strides(scale, m, n)
        desc.zero_row_stride, desc.zero_col_stride = _matrix_strides(zero, m, n)
        desc.qmin, desc.qmax = float(options["qmin"]), float(options["qmax"])
    elif kind == _abi.Q_ABSMAX_DYNAMIC:
        desc.qmin, desc.qmax, desc.half = float(options["qmin"]), float(options["qmax"]), options["half"]
    elif kind == _abi.Q_TRELLIS:
        (scale,) = quantizer_inputs
        assert scale.device == y.device, "the CUDA trellis quantizer requires Y, scale, and table on one CUDA device"
        # one scale per matrix of the batch, or one for all: anything finer goes through the per-stage engine
        per_batch, offsets = scale.to(y.dtype).reshape(-1), None
        if per_batch.numel() != 1:
            try:
                per_batch = scale.to(y.dtype).broadcast_to(*batch_shape, 1, 1, 1).reshape(-1).contiguous()
            except RuntimeError:
                return None
            offsets = torch.arange(per_batch.numel(), dtype=torch.int64, device=y.device)
        import quantizer_trellis

        table, index = quantizer_trellis.prepared_table(options["table"], y)
        keep += [per_batch, table, offsets, index]
        if index is not None:
            desc.table_distinct, desc.table_ids, desc.table_distinct_count = index[0].data_ptr(), index[1].data_ptr(), index[0].size(0)
        desc.scale, desc.scale_offsets, desc.table = per_batch.data_ptr(), _abi.ptr(offsets), table.data_ptr()
        desc.trellis_L, desc.trellis_K, desc.trellis_V = table.size(0).bit_length() - 1, options["K"], table.size(1)
        desc.tail_biting = int(bool(options["tail_biting"]))
        if codes is not None:
            desc.codes = codes.data_ptr()
    size = ctypes.c_size_t()
    _abi.check(lib.g2d_super_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)), "g2d_super_workspace_bytes")
    workspace = torch.empty(size.value, dtype=torch.uint8, device=y.device)
    desc.workspace, desc.workspace_bytes = workspace.data_ptr(), size.value
    with torch.cuda.device(y.device):
        _abi.check(lib.g2d_sweep_super_entry(ctypes.byref(desc), _abi.stream_of(y)), "g2d_sweep_super_entry")
    return y


def check_status(device=None) -> None:
    """Raise if a sweep on ``device`` since the last check hit a bounded wait that ran out inside a tensor-core kernel.

    The sweeps are asynchronous and never read device memory from the host; a failed wait (which a healthy GPU does
    not produce) turns the output into NaN and sets the device's status word.  This call waits for the device and
    reads the word, so a pipeline can run many layers and check once."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _abi.check_status(device, "gptq_2d")


def gptq_2d_forced(x: torch.Tensor, l: torch.Tensor, u: torch.Tensor, z: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Teacher-forced replay for parity checks: commit the given values ``z`` instead of rounding and return
    ``(z, y_pre)``, ``y_pre`` holding the value every entry had at the moment it would have been rounded."""
    y, m, n, batch_shape = _prepare_output(x, l, u, False)
    y_pre = torch.empty_like(y)
    if y.numel() == 0:
        return y, y_pre
    forced = z.expand_as(y).contiguous()
    _sweep_fused(y, l, u, batch_shape, dict(kind=_abi.Q_FORCED), (), forced_z=forced, y_pre=y_pre)
    return y, y_pre


# --------------------------------------------------------------------------------------------------------
# generic engine: an arbitrary Python quantizer per stage
# --------------------------------------------------------------------------------------------------------

def _sweep_generic(y, l, u, batch_shape, quantizer, quantizer_inputs, super_entry_shape, inner_block_size, outer_block_size):
    m, n = y.shape[-2:]
    p, q = super_entry_shape or (1, 1)
    lib = _abi.library()
    batch = batch_shape.numel()
    l, u = _row_major(l), _row_major(u)
    l_off, u_off = _abi.batch_offsets(l, batch_shape), _abi.batch_offsets(u, batch_shape)
    c = torch.zeros_like(y)  # running buffer C = L E
    e = torch.empty_like(y)  # errors of every finished entry
    lanes = min(m // p, n // q)
    z_scratch = y.new_empty(batch * lanes * p * q)
    stages = m // p + n // q - 1
    # the reference's clamping rules (gptq_2d.py:1327-1329)
    inner = inner_block_size if 0 < inner_block_size <= stages else stages
    outer = outer_block_size if inner < outer_block_size < stages else inner

    desc = _abi.StageDesc()
    desc.dtype, desc.p, desc.q = _abi.dtype_code(y.dtype), p, q
    desc.batch, desc.m, desc.n = batch, m, n
    desc.y, desc.c, desc.e = y.data_ptr(), c.data_ptr(), e.data_ptr()
    desc.l, desc.u, desc.l_offsets, desc.u_offsets = l.data_ptr(), u.data_ptr(), _abi.ptr(l_off), _abi.ptr(u_off)
    y_flat = y.flatten(start_dim=-2)  # live, storage-sharing
    stream = _abi.stream_of(y)
    ref = ctypes.byref(desc)

    with torch.cuda.device(y.device):
        for outer_start in range(0, stages, outer):
            outer_stop = min(outer_start + outer, stages)
            for s0 in range(outer_start, outer_stop, inner):
                s1 = min(s0 + inner, outer_stop)
                for s in range(s0, s1):
                    flat = _antidiagonal_slices(m=m, n=n, s=s, super_entry_shape=(p, q))[2]
                    selection: _Selection = flat
                    if super_entry_shape is not None:
                        selection = functools.partial(_super_entries, antidiagonal_slice=flat, n=n, super_entry_shape=(p, q))
                    selected = selection(y_flat) if callable(selection) else y_flat[..., selection]
                    z = z_scratch[:selected.numel()].view(selected.shape)
                    quantizer(y_flat, selection, *quantizer_inputs, out=z)
                    _abi.check(lib.g2d_stage_push(ref, z.data_ptr(), s, s1, stream), "g2d_stage_push")
                if s1 < outer_stop:
                    _abi.check(lib.g2d_stage_flush(ref, s0, s1, outer_stop, stream), "g2d_stage_flush")
            if outer_stop < stages:
                _abi.check(lib.g2d_stage_flush(ref, outer_start, outer_stop, stages, stream), "g2d_stage_flush")
    return y


def _run(x, l, u, quantizer, super_entry_shape, inner_block_size, outer_block_size, inplace, quantizer_inputs):
    y, m, n, batch_shape = _prepare_output(x, l, u, inplace, super_entry_shape or (1, 1))
    if y.numel() == 0:
        return y
    options = _fusable(quantizer, quantizer_inputs, super_entry_shape)
    if options is not None and not options["super"]:
        return _sweep_fused(y, l, u, batch_shape, options, quantizer_inputs)
    if options is not None and _sweep_super(y, l, u, batch_shape, options, quantizer_inputs, super_entry_shape, inner_block_size, outer_block_size) is not None:
        return y
    return _sweep_generic(y, l, u, batch_shape, quantizer, quantizer_inputs, super_entry_shape, inner_block_size, outer_block_size)


# --------------------------------------------------------------------------------------------------------
# public API
# --------------------------------------------------------------------------------------------------------

@torch.no_grad()
def gptq_2d(
    x: torch.Tensor, l: torch.Tensor, u: torch.Tensor, *,
    quantizer: Callable = round_quantizer, inner_block_size: int = 32, outer_block_size: int = 512,
    inplace: bool = False, quantizer_inputs: tuple[torch.Tensor, ...] = (),
) -> torch.Tensor:
    """Round ``x [*B, m, n]`` under the feedback factors ``l [*Bl, m, m]`` (unit lower) and ``u [*Bu, n, n]`` (unit upper).

    Same contract as the reference's ``gptq_2d`` (gptq_2d.py:1379-1418).  Only the entries of l below and of u above
    the diagonal are read.  ``quantizer(y_flat, antidiagonal_slice, *quantizer_inputs, out=z)`` receives live Y
    ``[*batch, m*n]`` whose earlier antidiagonals are already quantized, and must fill the contiguous
    ``out [*batch, antidiag_len]``.  Quantizers of this package are fused into the sweep kernels instead of being
    called; then the block sizes only matter to the generic engine (the result does not depend on them).
    ``inner_block_size`` outside ``1..m+n-1`` selects one block, ``outer_block_size`` outside
    ``inner_block_size+1..m+n-2`` single-level blocking.
    """
    return _run(x, l, u, quantizer, None, inner_block_size, outer_block_size, inplace, quantizer_inputs)


@torch.no_grad()
def gptq_2d_super_entry(
    x: torch.Tensor, l: torch.Tensor, u: torch.Tensor, *,
    quantizer: Callable = round_quantizer_super_entry, super_entry_shape: tuple[int, int] = (1, 1),
    inner_block_size: int = 8, outer_block_size: int = 64, inplace: bool = False,
    quantizer_inputs: tuple[torch.Tensor, ...] = (),
) -> torch.Tensor:
    """GPTQ-2D over jointly rounded ``p x q`` super-entries (the reference's gptq_2d.py:1422-1447).

    ``quantizer(y_flat, select, *quantizer_inputs, out=z)`` gets a selector that views any ``[..., m*n]`` tensor as
    the ``[..., d, p, q]`` super-entries of the current coarse antidiagonal.  l and u have implicit identity
    ``p x p`` / ``q x q`` diagonal blocks: only entries below / above those blocks are read.
    """
    return _run(x, l, u, quantizer, tuple(super_entry_shape), inner_block_size, outer_block_size, inplace, quantizer_inputs)


@torch.no_grad()
def gptq_2d_torch(x, l, u, *, quantizer: Callable = round_quantizer, inplace: bool = False, quantizer_inputs=()):
    """The reference's unblocked sweep (gptq_2d.py:1197-1236) by name: here the CUDA generic engine with one block."""
    y, m, n, batch_shape = _prepare_output(x, l, u, inplace)
    if y.numel() == 0:
        return y
    return _sweep_generic(y, l, u, batch_shape, quantizer, quantizer_inputs, None, 0, 0)


@torch.no_grad()
def gptq_2d_super_entry_torch(x, l, u, *, quantizer: Callable = round_quantizer_super_entry, super_entry_shape=(1, 1),
                              inplace: bool = False, quantizer_inputs=()):
    """The reference's unblocked super-entry sweep (gptq_2d.py:1240-1292) by name, on the CUDA generic engine."""
    y, m, n, batch_shape = _prepare_output(x, l, u, inplace, tuple(super_entry_shape))
    if y.numel() == 0:
        return y
    return _sweep_generic(y, l, u, batch_shape, quantizer, quantizer_inputs, tuple(super_entry_shape), 0, 0)


direct_2d = gptq_2d_torch  # gptq_2d.py:1123: the same result by dense updates; one engine serves both names here
direct_2d_super_entry = gptq_2d_super_entry_torch  # gptq_2d.py:1155


class _GraphedSweep:
    """A captured sweep and its private static buffers (the reference's capture_gptq_2d, gptq_2d.py:1451-1564)."""

    def __init__(self, run: Callable, inputs: tuple[torch.Tensor, ...], inplace: bool):
        self.inplace = inplace
        self.names = ("X", "L", "U", *(f"quantizer input {i}" for i in range(len(inputs) - 3)))
        self.expected = tuple((t.shape, t.dtype, t.device) for t in inputs)
        self.run = run
        self.graph = None
        x = inputs[0]
        if any(t.numel() == 0 for t in inputs[:3]):
            run(x=inputs[0], l=inputs[1], u=inputs[2], quantizer_inputs=inputs[3:])  # validates; no CUDA work to capture
            return
        self.static = tuple(t.detach().clone(memory_format=torch.contiguous_format) for t in inputs)
        with torch.cuda.device(x.device):
            side = torch.cuda.Stream(device=x.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):  # warm up outside the capture (kernel attributes, allocator pools)
                    run(x=self.static[0], l=self.static[1], u=self.static[2], quantizer_inputs=self.static[3:])
                self.static[0].copy_(x)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cuda_graph=self.graph, stream=side):
                self.result = run(x=self.static[0], l=self.static[1], u=self.static[2], quantizer_inputs=self.static[3:])

    def _validate(self, tensors) -> None:
        assert len(tensors) == len(self.expected), f"expected {len(self.expected) - 3} quantizer inputs"
        for name, tensor, (shape, dtype, device) in zip(self.names, tensors, self.expected):
            assert tensor.shape == shape, f"{name} shape must match its capture example"
            assert tensor.dtype == dtype, f"{name} dtype must match its capture example"
            assert tensor.device == device, f"{name} device must match its capture example"
        if self.inplace:
            assert tensors[0].is_contiguous(), "inplace=True requires contiguous X"

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, l: torch.Tensor, u: torch.Tensor, *quantizer_inputs: torch.Tensor) -> torch.Tensor:
        tensors = (x, l, u, *quantizer_inputs)
        self._validate(tensors)
        if self.graph is None:
            return self.run(x=x, l=l, u=u, quantizer_inputs=quantizer_inputs)
        for static, tensor in zip(self.static, tensors):
            static.copy_(tensor)
        self.graph.replay()
        if self.inplace:
            x.copy_(self.result)
            return x
        return self.result.clone()


@torch.no_grad()
def capture_gptq_2d(
    x: torch.Tensor, l: torch.Tensor, u: torch.Tensor, *,
    quantizer: Callable | None = None, super_entry_shape: tuple[int, int] | None = None,
    inner_block_size: int | None = None, outer_block_size: int | None = None, inplace: bool = False,
    quantizer_inputs: tuple[torch.Tensor, ...] = (),
) -> Callable[..., torch.Tensor]:
    """Capture one sweep in a CUDA graph and return ``replay(x, l, u, *quantizer_inputs)``.

    ``gptq_2d`` is captured, or ``gptq_2d_super_entry`` when ``super_entry_shape`` is given; options left as None
    keep that function's defaults.  Replay inputs must match the examples' shapes, dtypes and devices; they are
    copied into private static buffers.  Out-of-place replays return a fresh copy of the result, in-place replays
    copy it back into the caller's contiguous X and return that tensor.  A replay object owns its buffers and
    must be used sequentially.  A Python quantizer runs during warm-up and capture only.
    """
    _validate_inputs(x, l, u, inplace, True, super_entry_shape or (1, 1))
    assert all(t.is_cuda and t.device == x.device for t in quantizer_inputs), "quantizer inputs must be CUDA tensors on the same device as X"
    options = dict(quantizer=quantizer, super_entry_shape=super_entry_shape, inner_block_size=inner_block_size, outer_block_size=outer_block_size)
    run = functools.partial(
        gptq_2d if super_entry_shape is None else gptq_2d_super_entry, inplace=inplace,
        **{name: value for name, value in options.items() if value is not None},
    )
    return _GraphedSweep(run, (x, l, u, *quantizer_inputs), inplace)
