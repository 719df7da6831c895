"""Packed codes of a rounded matrix: the storage format behind the dequantised floats the sweep returns.

The reference returns dequantised values only and notes that the code can be recovered from them
(quantizer_trellis.py:11-14); for the affine quantizer (quantizer_int.py:63-83) the code of an entry is
``rint(z / scale + zero_point)``.  ``pack_codes`` forms ``code - qmin`` as ``bits``-bit unsigned fields, packed
little-endian along each row (entry ``j`` at the bits ``j * bits ...`` of the row's byte string, rows padded to whole
bytes); ``unpack_codes`` returns ``(code + qmin - zero_point) * scale``, bit for bit the value the quantizer produced.

Trellis codes are stored as the bit strings of their paths (``trellis_quantize_packed``, ``trellis_decode``,
``gptq_2d_trellis_packed``): the ``K V`` bits each step shifts into the state, most significant bit first, preceded by
the ``L - K V`` upper bits of the first state unless the path is tail-biting; bit ``i`` of a string is bit ``i % 8`` of
byte ``i // 8``.  A tail-biting sequence of ``T`` weights takes ``T K / 8`` bytes (64 for 256 weights at 2 bits).
CUDA only, like the rest of the package.
"""
from __future__ import annotations

import torch

import _abi


def _operands(m: int, n: int, scale: torch.Tensor, zero_point: torch.Tensor, dtype, device):
    out = []
    for name, t in (("scale", scale), ("zero_point", zero_point)):
        t = torch.as_tensor(t, dtype=dtype, device=device)
        assert t.dim() <= 2, f"{name} must broadcast to the matrix"
        t = torch.broadcast_to(t, (m, n))
        out.append((t, t.stride(0), t.stride(1)))
    return out


@torch.no_grad()
def pack_codes(z: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, *, qmin: float, bits: int) -> torch.Tensor:
    """``uint8 [m, ceil(n * bits / 8)]`` codes of the rounded matrix ``z [m, n]`` (float32 or float64, CUDA, contiguous)."""
    assert z.dim() == 2 and z.is_cuda and z.is_contiguous(), "expected a contiguous CUDA matrix"
    assert 1 <= bits <= 8, "bits must be between 1 and 8"
    m, n = z.shape
    row_bytes = (n * bits + 7) // 8
    codes = torch.empty(m, row_bytes, dtype=torch.uint8, device=z.device)
    if m == 0 or n == 0:
        return codes
    (s, srs, scs), (o, ors, ocs) = _operands(m, n, scale, zero_point, z.dtype, z.device)
    with torch.cuda.device(z.device):
        _abi.check(_abi.library().g2d_pack_codes(_abi.dtype_code(z.dtype), m, n, z.data_ptr(), s.data_ptr(), srs, scs, o.data_ptr(), ors, ocs,
                                                 float(qmin), bits, codes.data_ptr(), row_bytes, _abi.stream_of(z)), "g2d_pack_codes")
    return codes


@torch.no_grad()
def unpack_codes(codes: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, *, qmin: float, bits: int, n: int,
                 dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The dequantised matrix ``[m, n]`` of ``codes [m, row_bytes]`` (uint8, CUDA, contiguous)."""
    assert codes.dim() == 2 and codes.is_cuda and codes.is_contiguous() and codes.dtype == torch.uint8, "expected contiguous CUDA uint8 codes"
    assert 1 <= bits <= 8, "bits must be between 1 and 8"
    m, row_bytes = codes.shape
    assert row_bytes >= (n * bits + 7) // 8, "rows of codes are too short for n entries"
    z = torch.empty(m, n, dtype=dtype, device=codes.device)
    if m == 0 or n == 0:
        return z
    (s, srs, scs), (o, ors, ocs) = _operands(m, n, scale, zero_point, dtype, codes.device)
    with torch.cuda.device(codes.device):
        _abi.check(_abi.library().g2d_unpack_codes(_abi.dtype_code(dtype), m, n, codes.data_ptr(), row_bytes, s.data_ptr(), srs, scs, o.data_ptr(),
                                                   ors, ocs, float(qmin), bits, z.data_ptr(), _abi.stream_of(codes)), "g2d_unpack_codes")
    return z


def trellis_code_bytes(T: int, L: int, K: int, V: int, tail_biting: bool) -> int:
    """Bytes of one stored path of ``T`` weights."""
    import ctypes

    out = ctypes.c_int64()
    _abi.check(_abi.library().g2d_trellis_code_bytes(T, L, K, V, int(bool(tail_biting)), ctypes.byref(out)), "g2d_trellis_code_bytes")
    return out.value


def _trellis_operands(x_shape, table: torch.Tensor, K: int, scale, dtype, device):
    num_states, V = table.shape
    assert num_states & (num_states - 1) == 0 and V <= 2 and K * V <= 8 and x_shape[-1] % V == 0, "unsupported trellis code"
    rows = 1
    for size in x_shape[:-1]:
        rows *= size
    scale = torch.ones((), dtype=dtype, device=device) if scale is None else torch.as_tensor(scale, dtype=dtype, device=device)
    return num_states.bit_length() - 1, V, rows, scale.broadcast_to(x_shape[:-1]).reshape(rows).contiguous(), table.to(device=device, dtype=dtype).contiguous()


@torch.no_grad()
def trellis_quantize_packed(x: torch.Tensor, table: torch.Tensor, K: int, tail_biting: bool = True, scale=None) -> tuple[torch.Tensor, torch.Tensor]:
    """Search the trellis paths closest to the sequences ``x [..., T]`` (the search of ``quantizer_trellis``) and return
    ``(scale * values [..., T], codes uint8 [..., bytes])``: the dequantised values and the stored paths."""
    import ctypes

    assert x.is_cuda and x.dtype in (torch.float32, torch.float64), "expected float32 or float64 CUDA sequences"
    T = x.size(-1)
    L, V, rows, scale, table = _trellis_operands(x.shape, table, K, scale, x.dtype, x.device)
    nbytes = trellis_code_bytes(T, L, K, V, tail_biting)
    values = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    codes = torch.empty(*x.shape[:-1], nbytes, dtype=torch.uint8, device=x.device)
    if rows == 0:
        return values, codes
    lib, code = _abi.library(), _abi.dtype_code(x.dtype)
    size = ctypes.c_size_t()
    _abi.check(lib.g2d_trellis_workspace_bytes(code, rows, T, L, K, V, ctypes.byref(size)), "g2d_trellis_workspace_bytes")
    workspace = torch.empty(size.value, dtype=torch.uint8, device=x.device)
    flat = x.reshape(rows, T).contiguous()
    with torch.cuda.device(x.device):
        _abi.check(lib.g2d_trellis_quantize_packed(code, rows, T, flat.data_ptr(), table.data_ptr(), L, K, V, int(bool(tail_biting)), scale.data_ptr(),
                                                   values.data_ptr(), codes.data_ptr(), workspace.data_ptr(), size.value, _abi.stream_of(x)),
                   "g2d_trellis_quantize_packed")
    return values, codes


@torch.no_grad()
def trellis_decode(codes: torch.Tensor, table: torch.Tensor, K: int, T: int, tail_biting: bool = True, scale=None,
                   dtype: torch.dtype = torch.float32, return_states: bool = False):
    """``scale * values [..., T]`` of stored paths ``codes [..., bytes]`` (and the int64 states ``[..., T / V]``)."""
    assert codes.is_cuda and codes.dtype == torch.uint8 and codes.is_contiguous(), "expected contiguous CUDA uint8 codes"
    shape = (*codes.shape[:-1], T)
    L, V, rows, scale, table = _trellis_operands(shape, table, K, scale, dtype, codes.device)
    assert codes.size(-1) == trellis_code_bytes(T, L, K, V, tail_biting), "codes have the wrong number of bytes per sequence"
    values = torch.empty(shape, dtype=dtype, device=codes.device)
    states = torch.empty(*shape[:-1], T // V, dtype=torch.int64, device=codes.device) if return_states else None
    if rows:
        with torch.cuda.device(codes.device):
            _abi.check(_abi.library().g2d_trellis_decode(_abi.dtype_code(dtype), rows, T, codes.data_ptr(), table.data_ptr(), L, K, V,
                                                         int(bool(tail_biting)), scale.data_ptr(), values.data_ptr(), _abi.ptr(states),
                                                         _abi.stream_of(codes)), "g2d_trellis_decode")
    return (values, states) if return_states else values


@torch.no_grad()
def gptq_2d_trellis_packed(x: torch.Tensor, l: torch.Tensor, u: torch.Tensor, scale: torch.Tensor, *, table: torch.Tensor, K: int,
                           super_entry_shape: tuple[int, int], tail_biting: bool = True, inner_block_size: int = 8,
                           outer_block_size: int = 64) -> tuple[torch.Tensor, torch.Tensor]:
    """``gptq_2d_super_entry`` under the trellis quantizer that also returns the stored paths: ``(Z [*B, m, n],
    codes uint8 [*B, m / p, n / q, bytes])``; super-entry ``(i, j)``, read row by row, is the sequence of ``codes[..., i, j, :]``
    and ``trellis_decode`` gives back its part of Z bit for bit.  ``scale`` is one value, or one per matrix of the batch."""
    import gptq_2d as engine

    p, q = super_entry_shape
    y, m, n, batch_shape = engine._prepare_output(x, l, u, False, (p, q))
    V = table.size(1)
    nbytes = trellis_code_bytes(p * q, table.size(0).bit_length() - 1, K, V, tail_biting)
    codes = torch.zeros(*batch_shape, m // p, n // q, nbytes, dtype=torch.uint8, device=x.device)
    if y.numel() == 0:
        return y, codes
    options = dict(kind=_abi.Q_TRELLIS, table=table, K=K, tail_biting=tail_biting, super=True)
    done = engine._sweep_super(y, l, u, batch_shape, options, (scale,), (p, q), inner_block_size, outer_block_size, codes=codes)
    assert done is not None, "scale must be one value or one value per matrix of the batch"
    return y, codes


def pack_symmetric(matrix: torch.Tensor) -> torch.Tensor:
    """The lower triangle of a symmetric matrix ``[n, n]`` as ``n (n + 1) / 2`` values, row by row: half the bytes to move
    from host memory.  Runs wherever the tensor lives (on the host for a matrix that is about to travel)."""
    n = matrix.size(0)
    rows, cols = torch.tril_indices(n, n, device=matrix.device)
    return matrix[rows, cols].contiguous()


@torch.no_grad()
def unpack_symmetric(packed: torch.Tensor, n: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """The full symmetric CUDA matrix ``[n, n]`` of a packed lower triangle (``pack_symmetric``)."""
    assert packed.is_cuda and packed.is_contiguous() and packed.numel() == n * (n + 1) // 2, "expected n (n + 1) / 2 contiguous CUDA values"
    out = torch.empty(n, n, dtype=packed.dtype, device=packed.device) if out is None else out
    assert out.shape == (n, n) and out.is_contiguous() and out.dtype == packed.dtype and out.device == packed.device
    with torch.cuda.device(packed.device):
        _abi.check(_abi.library().g2d_symmetric_from_packed(_abi.dtype_code(packed.dtype), n, packed.data_ptr(), out.data_ptr(), _abi.stream_of(packed)),
                   "g2d_symmetric_from_packed")
    return out
