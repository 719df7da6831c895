"""Feedback factors of the Kronecker-factored Hessian on B200: ``ldl_of_inverse`` and ``feedback_factors``.

Same functions as the reference's gptq_2d_reference.py:41-66, which call ``torch.linalg.cholesky`` and
``solve_triangular``; here one hand-written CUDA pipeline (``csrc/g2d_factors.cu``): blocked reverse-order Cholesky,
blocked triangular inverse, normalisation by the diagonal blocks.
"""
from __future__ import annotations

import ctypes

import torch

import _abi


@torch.no_grad()
def ldl_of_inverse(M: torch.Tensor, size: int = 1, check: bool = True) -> torch.Tensor:
    """Unit lower (block) triangular L with ``M^{-1} = L Lambda L^T``, Lambda block diagonal with ``size x size``
    blocks, for a symmetric positive definite CUDA matrix ``M [n, n]`` (float32 or float64), without forming the inverse.

    With ``check`` (the default) the call waits for the result and raises ``torch.linalg.LinAlgError`` if a pivot was
    not positive, as ``torch.linalg.cholesky`` would; ``check=False`` keeps the call asynchronous."""
    assert M.dim() == 2 and M.size(0) == M.size(1), "expected a square matrix"
    assert M.is_cuda, "the CUDA factor preparation requires a CUDA tensor (there is no CPU path)"
    n = M.size(0)
    assert size > 0 and n % size == 0, "the block size must divide the matrix size"
    out = torch.empty(n, n, dtype=M.dtype, device=M.device)
    if n == 0:
        return out
    lib = _abi.library()
    code = _abi.dtype_code(M.dtype)
    work = M.clone(memory_format=torch.contiguous_format)  # the kernels factor in place
    need = ctypes.c_size_t()
    _abi.check(lib.g2d_ldl_workspace_bytes(code, n, ctypes.byref(need)), "g2d_ldl_workspace_bytes")
    workspace = torch.empty(need.value, dtype=torch.uint8, device=M.device)
    flag = torch.zeros(1, dtype=torch.int32, device=M.device)
    with torch.cuda.device(M.device):
        _abi.check(lib.g2d_ldl_of_inverse(code, n, work.data_ptr(), size, out.data_ptr(), flag.data_ptr(), workspace.data_ptr(),
                                          need.value, _abi.stream_of(M)), "g2d_ldl_of_inverse")
    if check:
        pivot = int(flag.item())
        if pivot:
            raise torch.linalg.LinAlgError(f"ldl_of_inverse: the matrix is not positive definite (pivot {pivot} is not positive)")
    return out


def feedback_factors(A: torch.Tensor, B: torch.Tensor, super_entry_shape: tuple[int, int] = (1, 1)) -> tuple[torch.Tensor, torch.Tensor]:
    """L and U with ``G^{-1} = L Lambda_L L^T`` and ``H^{-1} = U^T Lambda_U U`` for the Grams ``G = A^T A`` and
    ``H = B B^T``, with ``p x p`` and ``q x q`` identity diagonal blocks for ``p x q`` super-entries."""
    p, q = super_entry_shape
    return ldl_of_inverse(A.t() @ A, size=p), ldl_of_inverse(B @ B.t(), size=q).t()
