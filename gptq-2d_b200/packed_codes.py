"""Packed integer codes of a rounded matrix: the storage format behind the dequantised floats the sweep returns.

The reference returns dequantised values only and notes that the code can be recovered from them
(quantizer_trellis.py:11-14); for the affine quantizer (quantizer_int.py:63-83) the code of an entry is
``rint(z / scale + zero_point)``.  ``pack_codes`` forms ``code - qmin`` as ``bits``-bit unsigned fields, packed
little-endian along each row (entry ``j`` at the bits ``j * bits ...`` of the row's byte string, rows padded to whole
bytes); ``unpack_codes`` returns ``(code + qmin - zero_point) * scale``, bit for bit the value the quantizer produced.
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
