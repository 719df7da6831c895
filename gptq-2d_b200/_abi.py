"""ctypes binding of ``libgptq2d_b200.so`` (the C ABI declared in ``include/gptq2d_b200.h``).

The library is compiled in-tree by ``csrc/build.py``.  There is no fallback: if it is missing or a
call returns an error status, a ``RuntimeError`` says so.  Every call launches on PyTorch's current
CUDA stream of the tensors' device, so calls order with PyTorch's own work and can be captured in a
CUDA graph.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "csrc", "libgptq2d_b200.so")
ABI_VERSION = 2

F32, F64 = 0, 1
FP16, BF16 = 0, 1
Q_ROUND, Q_AFFINE, Q_ABSMAX_DYNAMIC, Q_TRELLIS, Q_FORCED = 0, 1, 2, 3, 4

_vp, _i64, _i32, _dbl = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_double


class SweepDesc(ctypes.Structure):
    """Mirror of ``g2d_sweep_desc``."""
    _fields_ = [
        ("dtype", _i32), ("quant_kind", _i32),
        ("batch", _i64), ("m", _i64), ("n", _i64),
        ("y", _vp),
        ("l", _vp), ("l_offsets", _vp),
        ("u", _vp), ("u_offsets", _vp),
        ("scale", _vp), ("scale_offsets", _vp),
        ("zero", _vp), ("zero_offsets", _vp),
        ("scale_row_stride", _i64), ("scale_col_stride", _i64), ("zero_row_stride", _i64), ("zero_col_stride", _i64),
        ("qmin", _dbl), ("qmax", _dbl),
        ("forced_z", _vp), ("y_pre", _vp),
        ("workspace", _vp), ("workspace_bytes", ctypes.c_size_t),
        ("outer_tiles", _i32), ("reserved", _i32),
        ("status", _vp),
    ]


class SuperDesc(ctypes.Structure):
    """Mirror of ``g2d_super_desc``."""
    _fields_ = [
        ("dtype", _i32), ("quant_kind", _i32), ("p", _i32), ("q", _i32), ("inner_block", _i32), ("outer_block", _i32),
        ("batch", _i64), ("m", _i64), ("n", _i64),
        ("y", _vp),
        ("l", _vp), ("l_offsets", _vp),
        ("u", _vp), ("u_offsets", _vp),
        ("lead_count", _i32), ("half", _i32),
        ("lead_size", _i64 * 4), ("lead_factor", _vp * 4),
        ("scale", _vp), ("scale_offsets", _vp),
        ("zero", _vp), ("zero_offsets", _vp),
        ("scale_row_stride", _i64), ("scale_col_stride", _i64), ("zero_row_stride", _i64), ("zero_col_stride", _i64),
        ("qmin", _dbl), ("qmax", _dbl),
        ("table", _vp),
        ("trellis_L", _i32), ("trellis_K", _i32), ("trellis_V", _i32), ("tail_biting", _i32),
        ("codes", _vp),
        ("workspace", _vp), ("workspace_bytes", ctypes.c_size_t),
        ("table_distinct", _vp), ("table_ids", _vp), ("table_distinct_count", _i32), ("reserved", _i32),
    ]


class StageDesc(ctypes.Structure):
    """Mirror of ``g2d_stage_desc``."""
    _fields_ = [
        ("dtype", _i32), ("p", _i32), ("q", _i32), ("reserved", _i32),
        ("batch", _i64), ("m", _i64), ("n", _i64),
        ("y", _vp), ("c", _vp), ("e", _vp),
        ("l", _vp), ("l_offsets", _vp),
        ("u", _vp), ("u_offsets", _vp),
    ]


_SIGNATURES = {
    "g2d_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "g2d_abi_version": (ctypes.c_int, []),
    "g2d_sweep_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(SweepDesc), ctypes.POINTER(ctypes.c_size_t)]),
    "g2d_sweep_fused": (ctypes.c_int, [ctypes.POINTER(SweepDesc), _vp]),
    "g2d_sweep_fused_static": (ctypes.c_int, [ctypes.POINTER(SweepDesc), _vp]),
    "g2d_super_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(SuperDesc), ctypes.POINTER(ctypes.c_size_t)]),
    "g2d_sweep_super_entry": (ctypes.c_int, [ctypes.POINTER(SuperDesc), _vp]),
    "g2d_trellis_code_bytes": (ctypes.c_int, [_i32, _i32, _i32, _i32, _i32, ctypes.POINTER(_i64)]),
    "g2d_trellis_quantize_packed": (ctypes.c_int, [ctypes.c_int, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, ctypes.c_size_t, _vp]),
    "g2d_trellis_quantize_indexed": (ctypes.c_int, [ctypes.c_int, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp,
                                                    ctypes.c_size_t, _vp]),
    "g2d_trellis_decode": (ctypes.c_int, [ctypes.c_int, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "g2d_sweep_fused_profile": (ctypes.c_int, [ctypes.POINTER(SweepDesc), _vp, ctypes.POINTER(ctypes.c_double)]),
    "g2d_launch_count": (ctypes.c_ulonglong, []),
    "g2d_stage_push": (ctypes.c_int, [ctypes.POINTER(StageDesc), _vp, _i64, _i64, _vp]),
    "g2d_stage_flush": (ctypes.c_int, [ctypes.POINTER(StageDesc), _i64, _i64, _i64, _vp]),
    "g2d_affine_quantize": (ctypes.c_int, [ctypes.c_int, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _dbl, _dbl, _vp, _vp]),
    "g2d_affine_quantize_super_entry": (ctypes.c_int, [ctypes.c_int, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _dbl, _dbl, _vp, _vp]),
    "g2d_absmax_scale": (ctypes.c_int, [ctypes.c_int, _i64, _i64, _i64, _i64, _vp, _dbl, _dbl, ctypes.c_int, _vp, _vp]),
    "g2d_absmax_quantize_super_entry": (ctypes.c_int, [ctypes.c_int, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _i64, _i64, _vp, _dbl, _dbl, ctypes.c_int, _vp, _vp]),
    "g2d_trellis_workspace_bytes": (ctypes.c_int, [ctypes.c_int, _i64, _i32, _i32, _i32, _i32, ctypes.POINTER(ctypes.c_size_t)]),
    "g2d_trellis_quantize": (ctypes.c_int, [ctypes.c_int, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, ctypes.c_size_t, _vp]),
    "g2d_ldl_workspace_bytes": (ctypes.c_int, [ctypes.c_int, _i64, ctypes.POINTER(ctypes.c_size_t)]),
    "g2d_ldl_of_inverse": (ctypes.c_int, [ctypes.c_int, _i64, _vp, _i32, _vp, _vp, _vp, ctypes.c_size_t, _vp]),
    "g2d_gram_workspace_bytes": (ctypes.c_int, [_i64, _i64, ctypes.POINTER(ctypes.c_size_t)]),
    "g2d_gram_accumulate": (ctypes.c_int, [_i64, _i64, _vp, ctypes.c_float, _vp, _vp, _vp, ctypes.c_size_t, _vp]),
    "g2d_pack_codes": (ctypes.c_int, [ctypes.c_int, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _i64, _i64, ctypes.c_double, _i32, _vp, _i64, _vp]),
    "g2d_unpack_codes": (ctypes.c_int, [ctypes.c_int, _i64, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _i64, ctypes.c_double, _i32, _vp, _vp]),
    "g2d_symmetric_from_packed": (ctypes.c_int, [ctypes.c_int, _i64, _vp, _vp, _vp]),
    "g2d_ldl_of_inverse_pair": (ctypes.c_int, [ctypes.c_int, _i64, _vp, _i32, _vp, _vp, ctypes.c_size_t,
                                               _i64, _vp, _i32, _vp, _vp, ctypes.c_size_t, _vp, _vp]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)
_LIB = None


def library() -> ctypes.CDLL:
    """The loaded CUDA library; raises if it has not been built (there is no CPU fallback)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIBRARY_PATH):
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python {os.path.join(_HERE, 'csrc', 'build.py')}` "
                "(needs nvcc; the library targets sm_100a). There is no CPU fallback."
            )
        lib = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        if lib.g2d_abi_version() != ABI_VERSION:
            raise RuntimeError(f"{LIBRARY_PATH} has ABI version {lib.g2d_abi_version()}, this binding expects {ABI_VERSION}: rebuild it")
        _LIB = lib
    return _LIB


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed: {library().g2d_status_string(status).decode()} (status {status})")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.float64:
        return F64
    raise AssertionError("expected float32 or float64")


def half_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return FP16
    if dtype == torch.bfloat16:
        return BF16
    raise AssertionError("the scale rounds to fp16 or bf16")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


_STATUS_WORDS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The device's persistent ``int32[1]`` status word.  The tensor-core kernels wait on hardware barriers with a
    time limit; a wait that runs out sets this word to -1 (the sweep also overwrites its output with NaN).  The
    library only ever sets it, so one read after many asynchronous calls tells whether all of them were sound."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _STATUS_WORDS:
        _STATUS_WORDS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return _STATUS_WORDS[index]


def check_status(device: torch.device, what: str = "gptq2d_b200") -> None:
    """Wait for the device and raise if any call since the last check reported a bounded wait that ran out."""
    word = status_word(device)
    value = int(word.item())
    if value != 0:
        word.zero_()
        raise RuntimeError(f"{what}: a bounded wait inside a tensor-core kernel ran out (status {value}); results since the last check are not valid")


def batch_offsets(x: torch.Tensor, batch_shape: torch.Size) -> torch.Tensor | None:
    """Element offset of each logical batch's matrix inside ``x``'s storage (``int64 [B]`` on the device),
    or None when there is a single matrix.  Broadcast dimensions get stride zero, so nothing is copied."""
    batch_size = batch_shape.numel()
    if batch_size == 1 and x.dim() == 2:
        return None
    padded = (1,) * (len(batch_shape) + 2 - x.dim()) + tuple(x.shape)
    strides = x.reshape(padded).expand(*batch_shape, *x.shape[-2:]).stride()[:-2]
    if all(stride == 0 for stride in strides):
        return None
    index = torch.arange(batch_size, dtype=torch.int64, device=x.device)
    offsets = torch.zeros_like(index)
    remaining = batch_size
    for size, stride in zip(batch_shape, strides):
        remaining //= size
        if stride:
            offsets += (index // remaining % size) * stride
    return offsets
