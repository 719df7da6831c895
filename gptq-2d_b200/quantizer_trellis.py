"""Bitshift trellis quantizer (QTIP) for super-entry GPTQ-2D on B200.

The public names of the reference's ``quantizer_trellis.py`` over one CUDA kernel (``csrc/g2d_trellis.cu``).
A trellis state is an L-bit window of a bitstream; each step shifts K*V new bits in and emits the V values
``table[state, :]``, so T values cost T*K bits.  The Viterbi search finds the bitstream whose values are closest to
the input; tail-biting makes it circular with two passes (quantizer_trellis.py:121-143 of the reference).  The
search returns exactly the reference's values and states: same cost arithmetic, first index on every tie.

``trellis_quantizer_super_entry_*`` round each super-entry, read row by row, as one sequence and write ``scale``
times its trellis values.  Nothing synchronizes with the host, so the quantizers run inside CUDA graphs.
"""
from __future__ import annotations

import ctypes
from collections.abc import Callable

import torch

import _abi


# ---- code tables (host-side PyTorch; one-time preparation) ---------------------------------------------------------

def one_mad(L: int = 16, device=None, dtype: torch.dtype | None = None) -> torch.Tensor:
    """1MAD code ``[2^L, 1]``: one multiply-add on the state, then the sum of its four bytes, centred and scaled in float32."""
    state = torch.arange(1 << L, dtype=torch.int64, device=device)
    mixed = (state * 34038481 + 76625530) & 0xFFFFFFFF
    total = sum((mixed >> (8 * byte)) & 255 for byte in range(4))
    divisor = torch.tensor(147.800537109375, dtype=torch.float32, device=device)  # a tensor, so the division is a true division
    return ((total - 510).float() / divisor)[:, None].to(dtype=dtype)


def three_inst(L: int = 16, device=None, dtype: torch.dtype | None = None) -> torch.Tensor:
    """3INST code ``[2^L, 1]``: one multiply-add, a mask and an xor give two fp16 bit patterns, which are summed in fp16."""
    state = torch.arange(1 << L, dtype=torch.int64, device=device)
    mixed = ((state * 89226354 + 64248484) & 0x8FFF8FFF) ^ 0x3B603B60
    bits = torch.stack((mixed >> 16, mixed & 0xFFFF), dim=-1)
    bits = torch.where(bits >= 1 << 15, bits - (1 << 16), bits).to(torch.int16)
    halves = bits.view(torch.float16)
    return (halves[:, 0] + halves[:, 1]).float()[:, None].to(dtype=dtype)


def _gaussian_codebook(size: int, seed: int = 0, samples: int = 1 << 16, iters: int = 25, device=None) -> torch.Tensor:
    """Seeded k-means codebook of the 2-D standard Gaussian with population standard deviation sqrt(15/16).

    The points are drawn on the CPU for every device and each cluster adds its points in their order, so the result
    does not depend on the device (the same recipe as quantizer_trellis.py:44-60 of the reference, whose default
    ``hyb()`` table this has to reproduce)."""
    generator = torch.Generator().manual_seed(seed)
    points = torch.randn(samples, 2, generator=generator).to(device)
    centers = torch.randn(size, 2, generator=generator).to(device)
    for _ in range(iters):
        owner = torch.cdist(points, centers).argmin(dim=1)
        counts = owner.bincount(minlength=size)
        sums = torch.segment_reduce(points[owner.argsort(stable=True), :], "sum", lengths=counts, axis=0)
        centers = torch.where(counts[:, None] > 0, sums / counts[:, None].clamp_min(1), centers)
    return centers / centers.std(correction=0) * (15 / 16) ** .5


def hyb(L: int = 16, tlut: torch.Tensor | None = None, seed: int = 0, device=None, dtype: torch.dtype | None = None) -> torch.Tensor:
    """HYB code ``[2^L, 2]``: hash each state to a row of the lookup table ``tlut [2^b, 2]`` and flip the sign of the
    first value by one more hash bit.  The default ``tlut`` is the seeded 2^9-row codebook above; pass a trained one to
    reproduce a QTIP checkpoint."""
    if tlut is None:
        tlut = _gaussian_codebook(1 << 9, seed=seed, device=device)
    bits = tlut.size(0).bit_length() - 1
    state = torch.arange(1 << L, dtype=torch.int64, device=tlut.device)
    hashed = state * (state + 1)
    table = tlut[(hashed >> (15 - bits)) & ((1 << bits) - 1), :]
    table[:, 0] *= 1 - 2 * ((hashed >> 15) & 1)
    return table.to(dtype=dtype)


# ---- an index of a code table: its distinct rows ----

_TABLE_INDEX: dict = {}
_INDEX_LIMIT = 2048  # distinct rows whose local costs fit shared memory beside the search's own buffers


def prepared_table(table: torch.Tensor, like: torch.Tensor) -> tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor] | None]:
    """The table in ``like``'s dtype and device, contiguous, and its index ``(distinct [D, V], ids int16 [2^L])`` when it has at
    most 2048 distinct rows and at most 2^16 states (else None).  The shipped codes have about a thousand distinct rows
    (``hyb``: 2^9 lookup rows times a sign), and the search is much faster when it knows them.  Both are remembered per
    table (keyed by its storage and version), so a sweep that calls the quantizer a thousand times prepares them once."""
    key = (table.data_ptr(), table._version, tuple(table.shape), table.dtype, table.device, like.dtype, like.device)
    if key not in _TABLE_INDEX:
        if len(_TABLE_INDEX) > 16:
            _TABLE_INDEX.clear()
        converted = table.to(like).contiguous()
        index = None
        if converted.is_cuda and 64 <= converted.size(0) <= 1 << 16:
            distinct, inverse = torch.unique(converted, dim=0, return_inverse=True)
            if distinct.size(0) <= _INDEX_LIMIT:
                index = (distinct.contiguous(), inverse.to(torch.int16).contiguous())
        _TABLE_INDEX[key] = (table, converted, index)  # the table itself is kept alive: its address is part of the key
    return _TABLE_INDEX[key][1:]


# ---- the search ------------------------------------------------------------------------------------------------------

def _trellis_quantize_cuda(
    x: torch.Tensor, table: torch.Tensor, K: int, tail_biting: bool, *,
    out: torch.Tensor, scale: torch.Tensor, states: torch.Tensor | None = None,
) -> None:
    """Write ``out [..., T] = scale[..., None] *`` the values of the trellis paths closest to ``x [..., T]``, and the
    states ``[..., T/V]`` (int64) into ``states`` if given; both contiguous."""
    num_states, V = table.shape
    T, shift = x.size(-1), K * V
    assert V <= 2 and shift <= 8 and T % V == 0, "the same sums need V <= 2, and a walk back holds 2^(K*V) <= 256 candidates"
    assert x.is_cuda and table.device == x.device and scale.device == x.device, (
        "the CUDA trellis quantizer requires Y, scale, and table on one CUDA device"
    )
    assert x.dtype in (torch.float32, torch.float64), "expected float32 or float64 sequences"
    x = x.reshape(-1, T).contiguous()
    rows = x.size(0)
    if rows == 0:
        return
    L = num_states.bit_length() - 1
    assert out.is_contiguous() and out.numel() == rows * T and out.dtype == x.dtype, "out must be contiguous [..., T] in x's dtype"
    scale = scale.to(x.dtype).broadcast_to(out.shape[:-1]).reshape(rows).contiguous()
    table, index = prepared_table(table, x)
    if states is not None:
        assert states.is_contiguous() and states.dtype == torch.int64 and states.numel() == rows * (T // V)
    lib = _abi.library()
    size = ctypes.c_size_t()
    code = _abi.dtype_code(x.dtype)
    _abi.check(lib.g2d_trellis_workspace_bytes(code, rows, T, L, K, V, ctypes.byref(size)), "g2d_trellis_workspace_bytes")
    # Power-of-two capacity: inside a captured sweep the antidiagonals grow, and a graph's memory pool reuses a
    # freed buffer only for requests that fit in it, so rounding up keeps the pool below twice the largest request.
    capacity = 1 << max(size.value - 1, 0).bit_length()
    workspace = torch.empty(capacity, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        if index is not None:
            distinct, ids = index
            _abi.check(lib.g2d_trellis_quantize_indexed(
                code, rows, T, x.data_ptr(), table.data_ptr(), L, K, V, int(bool(tail_biting)), scale.data_ptr(), out.data_ptr(),
                _abi.ptr(states), None, distinct.data_ptr(), distinct.size(0), ids.data_ptr(), workspace.data_ptr(), capacity,
                _abi.stream_of(x)), "g2d_trellis_quantize_indexed")
        else:
            _abi.check(lib.g2d_trellis_quantize(
                code, rows, T, x.data_ptr(), table.data_ptr(), L, K, V, int(bool(tail_biting)), scale.data_ptr(), out.data_ptr(),
                _abi.ptr(states), workspace.data_ptr(), capacity, _abi.stream_of(x)), "g2d_trellis_quantize")


def _trellis_quantize(x: torch.Tensor, table: torch.Tensor, K: int, tail_biting: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Values ``[..., T]`` and states ``[..., T/V]`` of the closest trellis paths (the return convention of the
    reference's ``_trellis_quantize_torch``, quantizer_trellis.py:121)."""
    V = table.size(1)
    values = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    states = torch.empty(*x.shape[:-1], x.size(-1) // V, dtype=torch.int64, device=x.device)
    _trellis_quantize_cuda(x, table, K, tail_biting, out=values, scale=x.new_ones(x.shape[:-1]), states=states)
    return values, states


def trellis_quantizer_super_entry_cuda(
    y_flat: torch.Tensor, select: Callable[[torch.Tensor], torch.Tensor], scale: torch.Tensor, *,
    out: torch.Tensor, table: torch.Tensor, K: int, tail_biting: bool = True,
) -> None:
    """Trellis-quantize the selected antidiagonal of super-entries into ``out [*batch, d, p, q]``.

    Each super-entry of ``select(y_flat) / scale``, read row by row, is one sequence, and ``out`` gets ``scale`` times
    its values.  ``scale`` broadcasts against the super-entries and is constant within each."""
    x = select(y_flat) / scale
    sequences = x.flatten(start_dim=-2)
    per_entry = scale.broadcast_to(x.shape)[..., 0, 0].to(x.dtype)
    _trellis_quantize_cuda(sequences, table, K, tail_biting, out=out.view(sequences.shape), scale=per_entry)


def _viterbi(x: torch.Tensor, table: torch.Tensor, K: int, init: torch.Tensor | None = None, final: torch.Tensor | None = None) -> torch.Tensor:
    """States ``[..., T/V]`` of the trellis path closest to ``x [..., T]`` (the reference's tested private ``_viterbi``,
    quantizer_trellis.py:82-118) for unconstrained paths.  The reference passes boolean state masks ``init`` / ``final``
    only to impose the two tail-biting constraints (:136-142); the CUDA search applies those itself
    (``_trellis_quantize(..., tail_biting=True)``), so arbitrary masks are not taken here."""
    assert init is None and final is None, "state masks are internal to the CUDA search: use _trellis_quantize(..., tail_biting=True)"
    return _trellis_quantize(x, table, K, False)[1]


# The reference's names: one CUDA implementation behind all of them.
_trellis_quantize_torch = _trellis_quantize
_trellis_quantize_triton = _trellis_quantize_cuda
trellis_quantizer_super_entry_torch = trellis_quantizer_super_entry_triton = trellis_quantizer_super_entry_cuda
