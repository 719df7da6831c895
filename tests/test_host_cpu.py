"""CPU-side checks: the C ABI library loads and exports what the header declares; host logic of the drop-in API."""
import ctypes
import functools
import os
import re

import pytest
import torch

from conftest import ROOT


def test_library_exports_every_declared_symbol():
    import _abi

    header = open(os.path.join(ROOT, "include", "gptq2d_b200.h")).read()
    declared = set(re.findall(r"\b(g2d_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_abi.LIBRARY_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(_abi.EXPORTED_SYMBOLS) == declared
    assert _abi.library().g2d_abi_version() == _abi.ABI_VERSION
    assert _abi.library().g2d_status_string(-2) == b"workspace missing, misaligned or too small"


def test_descriptor_layout_matches_header():
    import _abi

    # field order and C alignment rules give these sizes for the header's structs on LP64
    assert ctypes.sizeof(_abi.SweepDesc) == 8 + 3 * 8 + 9 * 8 + 4 * 8 + 2 * 8 + 2 * 8 + 2 * 8 + 8 + 8
    assert ctypes.sizeof(_abi.StageDesc) == 16 + 3 * 8 + 7 * 8
    assert ctypes.sizeof(_abi.SuperDesc) == 6 * 4 + 3 * 8 + 5 * 8 + 2 * 4 + 4 * 8 + 4 * 8 + 4 * 8 + 4 * 8 + 2 * 8 + 8 + 4 * 4 + 8 + 2 * 8 + 2 * 8 + 2 * 4


def test_cpu_tensors_are_rejected_not_emulated():
    import gptq_2d as G

    x, l, u = torch.randn(4, 6), torch.randn(4, 4), torch.randn(6, 6)
    with pytest.raises(AssertionError, match="must be CUDA tensors"):
        G.gptq_2d(x, l, u)
    with pytest.raises(AssertionError, match="must be CUDA tensors"):
        G.capture_gptq_2d(x, l, u)


def test_validation_messages():
    import gptq_2d as G

    x, l, u = torch.randn(4, 6), torch.randn(4, 4), torch.randn(6, 6)
    with pytest.raises(AssertionError, match="expected X="):
        G._validate_inputs(x, u, l, False, False)
    with pytest.raises(AssertionError, match="super-entry shape must divide"):
        G._validate_inputs(x, l, u, False, False, (3, 2))
    with pytest.raises(AssertionError, match="share dtype"):
        G._validate_inputs(x.double(), l, u, False, False)
    with pytest.raises(AssertionError, match="inplace=True requires"):
        G._validate_inputs(x, l[None].expand(2, 4, 4), u, True, False)
    assert G._validate_inputs(x[None], l[None].expand(3, 4, 4), u, False, False) == (4, 6, torch.Size([3]))


def test_antidiagonal_geometry():
    import gptq_2d as G

    for m, n, p, q in ((5, 7, 1, 1), (7, 5, 1, 1), (1, 9, 1, 1), (8, 12, 2, 4), (4, 64, 1, 32), (16, 16, 16, 16), (6, 6, 3, 2)):
        flat = torch.arange(m * n)
        matrix = flat.view(m, n)
        seen = torch.zeros(m * n, dtype=torch.int64)
        for s in range(m // p + n // q - 1):
            rows, cols, sl = G._antidiagonal_slices(m=m, n=n, s=s, super_entry_shape=(p, q))
            view = G._super_entries(flat, sl, n, (p, q))
            k = 0
            for ibar in range(rows.start, rows.stop):
                jbar = s - ibar
                assert cols.start <= jbar < cols.stop
                assert torch.equal(view[k], matrix[ibar * p:(ibar + 1) * p, jbar * q:(jbar + 1) * q])
                k += 1
            assert view.shape[0] == k
            seen[view.flatten()] += 1
        assert (seen == 1).all()


def test_fused_dispatch_recognition():
    import gptq_2d as G
    import quantizer_int as Q

    import quantizer_trellis as T

    t = torch.zeros(2, 2)
    # plain entries under the round and affine quantizers: the fused tile engine
    assert G._fusable(Q.round_quantizer, (), None) == {"kind": 0, "super": False}
    assert G._fusable(functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7), (t, t), None) == {"kind": 1, "qmin": -8, "qmax": 7, "super": False}
    assert G._fusable(functools.partial(functools.partial(Q.affine_quantizer_torch, qmin=-8), qmax=7), (t, t), None)["qmax"] == 7
    assert G._fusable(Q.affine_quantizer_super_entry_triton, (t, t), (1, 1)) == {"kind": 1, "qmin": -torch.inf, "qmax": torch.inf, "super": False}
    # larger super-entries and the joint quantizers: the library's super-entry sweep
    assert G._fusable(Q.affine_quantizer_super_entry_triton, (t, t), (2, 2))["super"] is True
    assert G._fusable(Q.round_quantizer_super_entry, (), (2, 4)) == {"kind": 0, "super": True}
    absmax = functools.partial(Q.int_abs_max_quantizer_triton, qmin=-8, qmax=7, dtype=torch.bfloat16)
    assert G._fusable(absmax, (), (1, 32)) == {"kind": 2, "qmin": -8, "qmax": 7, "half": 1, "super": True}
    assert G._fusable(absmax, (), None) is None
    assert G._fusable(functools.partial(Q.int_abs_max_quantizer_triton, qmin=-8, qmax=7, dtype=torch.float32), (), (1, 32)) is None
    table = torch.zeros(256, 2)
    trellis = G._fusable(functools.partial(T.trellis_quantizer_super_entry_triton, table=table, K=2), (t,), (16, 16))
    assert trellis["kind"] == 3 and trellis["K"] == 2 and trellis["tail_biting"] is True and trellis["super"] is True
    assert G._fusable(functools.partial(T.trellis_quantizer_super_entry_triton, table=table, K=2), (t,), (3, 5)) is None  # T % V
    assert G._fusable(functools.partial(T.trellis_quantizer_super_entry_triton, table=torch.zeros(256, 3), K=2), (t,), (3, 4)) is None
    # anything else: the per-stage engine calls it
    assert G._fusable(Q.affine_quantizer_triton, (t,), None) is None
    assert G._fusable(lambda *a, **k: None, (), None) is None
    assert G._fusable(functools.partial(Q.affine_quantizer_triton, t), (t, t), None) is None


def test_batch_offsets_follow_broadcasting():
    import _abi

    l = torch.zeros(1, 3, 4, 4)
    assert _abi.batch_offsets(l, torch.Size([2, 3])).tolist() == [0, 16, 32, 0, 16, 32]
    assert _abi.batch_offsets(torch.zeros(4, 4), torch.Size([])) is None
    assert _abi.batch_offsets(torch.zeros(4, 4), torch.Size([5])) is None  # fully broadcast
    assert _abi.batch_offsets(torch.zeros(2, 1, 4, 4), torch.Size([2, 3])).tolist() == [0, 0, 0, 16, 16, 16]
