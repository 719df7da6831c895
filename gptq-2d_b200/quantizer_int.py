"""INT quantizers for GPTQ-2D on B200: the public names of the reference's ``quantizer_int.py`` over CUDA kernels.

The affine quantizers write ``(clamp(round(y / scale + zero_point), qmin, qmax) - zero_point) * scale``
(round half to even, IEEE division) and need nonzero scales; ``int_abs_max_scale_*`` gives GPTQ's symmetric
per-row scales, and ``int_abs_max_quantizer_*`` rounds each row of a super-entry with a scale taken from its
current values.  The ``_torch`` and ``_triton`` names of the reference (quantizer_int.py:63, :86, :110, :120,
:208, :302, :388, :442) are kept so that callers need not change; here every one of them runs the same
hand-written CUDA kernel (``csrc/g2d_quantizers.cu``) and requires CUDA tensors.  ``gptq_2d`` recognises these
functions (also wrapped in ``functools.partial``) and fuses them into its sweep kernels.
"""
from __future__ import annotations

from collections.abc import Callable

import torch

import _abi


def round_quantizer(y_flat: torch.Tensor, antidiagonal_slice: slice, *, out: torch.Tensor) -> None:
    """Round the selected antidiagonal to the nearest integers (ties to even) into ``out``."""
    torch.round(y_flat[..., antidiagonal_slice], out=out)


def round_quantizer_super_entry(y_flat: torch.Tensor, select: Callable[[torch.Tensor], torch.Tensor], *, out: torch.Tensor) -> None:
    """Round the selected antidiagonal of super-entries to the nearest integers into ``out``."""
    torch.round(select(y_flat), out=out)


def _validate_affine_inputs(y_flat, scale, zero_point, out, qmin, qmax) -> torch.Size:
    """The checks of the reference (quantizer_int.py:38-60), with its messages; returns Y's batch shape."""
    assert qmin < qmax, "expected qmin < qmax"
    assert scale.dim() >= 2 and zero_point.dim() >= 2, "scale and zero point must have matrix dimensions"
    assert scale.shape[-2:] == zero_point.shape[-2:], "scale and zero point matrix shapes must match"
    assert scale.shape[-2:].numel() == y_flat.size(-1), "scale and zero point matrix shapes must match Y"
    assert scale.dtype == zero_point.dtype == y_flat.dtype, "scale, zero point, and Y must share dtype"
    assert scale.device == zero_point.device == y_flat.device, "scale, zero point, and Y must share device"
    batch_shape = y_flat.shape[:-1]
    assert torch.broadcast_shapes(scale.shape[:-2], zero_point.shape[:-2], batch_shape) == batch_shape, (
        "scale and zero point batch dimensions must broadcast to Y"
    )
    assert out.shape[:-1] == batch_shape and out.dtype == y_flat.dtype and out.device == y_flat.device, (
        "out must match Y's batch shape, dtype, and device"
    )
    return batch_shape


def _require_cuda(y_flat: torch.Tensor, *others: torch.Tensor) -> None:
    assert y_flat.is_cuda, "the CUDA quantizers require CUDA tensors (there is no CPU path)"
    assert y_flat.is_contiguous() and all(t.is_contiguous() for t in others), "the CUDA quantizers require contiguous Y, scale, zero point, and out"


def affine_quantizer_cuda(
    y_flat: torch.Tensor, antidiagonal_slice: slice, scale: torch.Tensor, zero_point: torch.Tensor, *,
    out: torch.Tensor, qmin: float = -torch.inf, qmax: float = torch.inf,
) -> None:
    """Affine-quantize one antidiagonal of ``y_flat [*batch, m*n]`` into the contiguous ``out [*batch, len]``.

    ``scale`` and ``zero_point`` are ``[*Bs, m, n]`` matrices whose batch dimensions broadcast to Y's.
    """
    batch_shape = _validate_affine_inputs(y_flat, scale, zero_point, out, qmin, qmax)
    _require_cuda(y_flat, scale, zero_point, out)
    start, stop, step = antidiagonal_slice.indices(y_flat.size(-1))
    count = max(0, -(-(stop - start) // step))
    assert out.shape == (*batch_shape, count), "out must match the selected antidiagonal"
    if out.numel() == 0:
        return
    with torch.cuda.device(y_flat.device):
        _abi.check(_abi.library().g2d_affine_quantize(
            _abi.dtype_code(y_flat.dtype), batch_shape.numel(), y_flat.size(-1), start, step, count,
            _abi.ptr(y_flat), _abi.ptr(scale), _abi.ptr(_abi.batch_offsets(scale, batch_shape)),
            _abi.ptr(zero_point), _abi.ptr(_abi.batch_offsets(zero_point, batch_shape)),
            float(qmin), float(qmax), _abi.ptr(out), _abi.stream_of(y_flat)), "g2d_affine_quantize")


def _selected_layout(select, source: torch.Tensor) -> tuple[torch.Tensor, int]:
    view = select(source)
    assert view.untyped_storage().data_ptr() == source.untyped_storage().data_ptr(), "select must return views"
    return view, view.storage_offset() - source.storage_offset()


def affine_quantizer_super_entry_cuda(
    y_flat: torch.Tensor, select: Callable[[torch.Tensor], torch.Tensor], scale: torch.Tensor, zero_point: torch.Tensor, *,
    out: torch.Tensor, qmin: float = -torch.inf, qmax: float = torch.inf,
) -> None:
    """Affine-quantize the selected antidiagonal of super-entries, entry by entry, into ``out [*batch, d, p, q]``.

    ``select`` must return views (as ``gptq_2d_super_entry``'s does); the kernel reads Y, scale and zero point
    through the views' strides.
    """
    batch_shape = _validate_affine_inputs(y_flat, scale, zero_point, out.flatten(start_dim=-3), qmin, qmax)
    _require_cuda(y_flat, scale, zero_point, out)
    y_view, first = _selected_layout(select, y_flat)
    s_view, s_first = _selected_layout(select, scale.flatten(start_dim=-2))
    z_view, z_first = _selected_layout(select, zero_point.flatten(start_dim=-2))
    assert y_view.stride()[-3:] == s_view.stride()[-3:] == z_view.stride()[-3:] and first == s_first == z_first, (
        "Y, scale, and zero point must share their layout"
    )
    assert out.shape == y_view.shape, "out must match the selected super-entries"
    d, p, q = y_view.shape[-3:]
    if out.numel() == 0:
        return
    with torch.cuda.device(y_flat.device):
        _abi.check(_abi.library().g2d_affine_quantize_super_entry(
            _abi.dtype_code(y_flat.dtype), batch_shape.numel(), y_flat.size(-1), first, d, p, q,
            y_view.stride(-3), y_view.stride(-2), y_view.stride(-1),
            _abi.ptr(y_flat), _abi.ptr(scale), _abi.ptr(_abi.batch_offsets(scale, batch_shape)),
            _abi.ptr(zero_point), _abi.ptr(_abi.batch_offsets(zero_point, batch_shape)),
            float(qmin), float(qmax), _abi.ptr(out), _abi.stream_of(y_flat)), "g2d_affine_quantize_super_entry")


def int_abs_max_scale_cuda(x: torch.Tensor, *, qmin: float, qmax: float, dtype: torch.dtype) -> torch.Tensor:
    """GPTQ's symmetric scale of each row of ``x [..., size]`` for the codes qmin..qmax: ``absmax / ((qmax - qmin) / 2)``
    rounded to the 16-bit ``dtype`` (through float32, ties to even) and returned in x's dtype as ``[..., 1]``;
    1 for a row of zeros.  Rows are read through a view when x's leading dimensions merge."""
    assert x.is_cuda, "the CUDA scale requires a CUDA tensor"
    assert qmin < qmax, "expected qmin < qmax"
    half = _abi.half_code(dtype)
    rows = x.reshape(-1, x.size(-1))
    out = x.new_empty(*x.shape[:-1], 1)
    if out.numel() == 0:
        return out
    with torch.cuda.device(x.device):
        _abi.check(_abi.library().g2d_absmax_scale(
            _abi.dtype_code(x.dtype), rows.size(0), rows.size(1), rows.stride(0), rows.stride(1), _abi.ptr(rows),
            float(qmin), float(qmax), half, _abi.ptr(out), _abi.stream_of(x)), "g2d_absmax_scale")
    return out


def int_abs_max_quantizer_cuda(
    y_flat: torch.Tensor, select: Callable[[torch.Tensor], torch.Tensor], *, out: torch.Tensor,
    qmin: float, qmax: float, dtype: torch.dtype,
) -> None:
    """Round each row of the selected super-entries to the integers qmin..qmax times a scale from its current
    values, ``absmax / ((qmax - qmin) / 2)`` rounded to ``dtype``, into ``out [*batch, d, p, q]``."""
    assert y_flat.is_cuda, "the CUDA quantizer requires CUDA tensors"
    assert y_flat.is_contiguous() and out.is_contiguous(), "the CUDA quantizer requires contiguous Y and out"
    view, first = _selected_layout(select, y_flat)
    assert out.shape == view.shape and out.dtype == view.dtype, "out must match the selected super-entries"
    assert qmin < qmax, "expected qmin < qmax and a scale in fp16 or bf16"
    half = _abi.half_code(dtype)
    d, p, q = view.shape[-3:]
    if out.numel() == 0:
        return
    with torch.cuda.device(y_flat.device):
        _abi.check(_abi.library().g2d_absmax_quantize_super_entry(
            _abi.dtype_code(y_flat.dtype), y_flat.shape[:-1].numel(), y_flat.size(-1), first, d, p, q,
            view.stride(-3), view.stride(-2), view.stride(-1), _abi.ptr(y_flat),
            float(qmin), float(qmax), half, _abi.ptr(out), _abi.stream_of(y_flat)), "g2d_absmax_quantize_super_entry")


# The reference's names: one CUDA implementation behind all of them.
affine_quantizer_torch = affine_quantizer_triton = affine_quantizer_cuda
affine_quantizer_super_entry_torch = affine_quantizer_super_entry_triton = affine_quantizer_super_entry_cuda
int_abs_max_scale_torch = int_abs_max_scale_triton = int_abs_max_scale_cuda
int_abs_max_quantizer_torch = int_abs_max_quantizer_triton = int_abs_max_quantizer_cuda
