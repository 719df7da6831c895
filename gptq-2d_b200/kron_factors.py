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
        if pivot < 0:
            raise RuntimeError("ldl_of_inverse: a bounded wait inside a tensor-core kernel ran out; the result is not valid")
        if pivot:
            raise torch.linalg.LinAlgError(f"ldl_of_inverse: the matrix is not positive definite (pivot {pivot} is not positive)")
    else:
        _PENDING.append((flag, ("the matrix",)))  # settled by check_pending(), like the pair call's flags
    return out


@torch.no_grad()
def accumulate_gram(h: torch.Tensor, x: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """``h += alpha * x.T @ x`` in place on the tensor cores, at float32 fidelity: the Hessian-factor accumulation that
    precedes ``ldl_of_inverse`` in a pipeline (``x [k samples, n channels]``, ``h [n, n]``, float32, CUDA, contiguous,
    ``n`` a multiple of 4).  The reference leaves this step to the caller (demo.ipynb:103-106)."""
    assert h.is_cuda and x.is_cuda and h.device == x.device, "the Gram accumulation requires CUDA tensors (there is no CPU path)"
    assert h.dtype == torch.float32 and x.dtype == torch.float32, "float32 only"
    assert x.dim() == 2 and h.shape == (x.size(1), x.size(1)) and h.is_contiguous() and x.is_contiguous(), "expected x [k, n] and h [n, n], contiguous"
    k, n = x.shape
    assert n % 4 == 0, "the channel count must be a multiple of 4"
    if n == 0 or k == 0:
        return h
    lib = _abi.library()
    need = ctypes.c_size_t()
    _abi.check(lib.g2d_gram_workspace_bytes(n, k, ctypes.byref(need)), "g2d_gram_workspace_bytes")
    workspace = torch.empty(need.value, dtype=torch.uint8, device=h.device)
    with torch.cuda.device(h.device):
        _abi.check(lib.g2d_gram_accumulate(n, k, x.data_ptr(), float(alpha), h.data_ptr(), _abi.status_word(h.device).data_ptr(),
                                           workspace.data_ptr(), need.value, _abi.stream_of(h)), "g2d_gram_accumulate")
    return h


def feedback_factors(A: torch.Tensor, B: torch.Tensor, super_entry_shape: tuple[int, int] = (1, 1)) -> tuple[torch.Tensor, torch.Tensor]:
    """L and U with ``G^{-1} = L Lambda_L L^T`` and ``H^{-1} = U^T Lambda_U U`` for the Grams ``G = A^T A`` and
    ``H = B B^T``, with ``p x p`` and ``q x q`` identity diagonal blocks for ``p x q`` super-entries."""
    p, q = super_entry_shape
    return ldl_of_inverse(A.t() @ A, size=p), ldl_of_inverse(B @ B.t(), size=q).t()


@torch.no_grad()
def gptq_d_sided(x: torch.Tensor, factors, *, quantizer=None, quantizer_inputs=(), super_entry_shape=(1, 1),
                 inner_block_size: int = 8, outer_block_size: int = 64, dense_row_factor: bool = False, **sweep_options) -> torch.Tensor:
    """N-factor (D-sided) rounding of an ``n_1 x ... x n_D`` tensor under one unit lower triangular factor per mode
    (Algorithm 4 of the paper; the reference's slow ``alg4``, gptq_2d_reference.py:269-294).

    The tensor is swept as ``n_1 ... n_{D-2}`` slabs ``[n_{D-1}, n_D]`` under ``(L_{D-1}, L_D^T)``; the leading modes
    couple the slabs through scaled additions of the finished slabs' residuals, mode by mode, so no factor larger than
    ``n_d x n_d`` is ever formed, and all slabs advance together along the hyper-anti-diagonals ``i_1 + ... + i_D = s``.
    ``quantizer`` is one of this package's quantizers as ``gptq_2d_super_entry`` takes it (default: rounding), applied to
    ``(1, ..., 1, p, q)`` super-entries of the last two modes; ``quantizer_inputs`` are its tensors for the
    ``[n_1 ... n_{D-2}, n_{D-1}, n_D]`` view (an affine scale is ``[..., n_{D-1}, n_D]``).

    ``dense_row_factor=True`` (or a quantizer the library does not know, or more than six modes) takes the other route:
    the two-sided sweep on ``[n_1 ... n_{D-1}, n_D]`` with the explicit Kronecker row factor
    ``kron(L_1, ..., L_{D-1})``, where ``quantizer`` follows ``gptq_2d`` on that matrix and ``sweep_options`` are passed on.
    """
    import functools

    import gptq_2d as engine
    from quantizer_int import round_quantizer, round_quantizer_super_entry

    factors = list(factors)
    assert x.dim() == len(factors) >= 1, "expected one factor per mode"
    assert all(f.shape == (k, k) for f, k in zip(factors, x.shape)), "factor d must be n_d x n_d"
    assert x.is_cuda and all(f.device == x.device and f.dtype == x.dtype for f in factors), "X and the factors must share a CUDA device and dtype"
    if x.numel() == 0:
        return x.clone()
    p, q = super_entry_shape
    structured = not dense_row_factor and not sweep_options and 3 <= x.dim() <= 6  # two modes: the two-sided engines below
    options = None
    if structured:
        chosen = quantizer if quantizer is not None else round_quantizer_super_entry
        if chosen is round_quantizer:
            chosen = round_quantizer_super_entry
        options = engine._fusable(chosen, quantizer_inputs, (p, q))
    if options is not None:
        lead = factors[:-2]
        m, n = x.shape[-2:]
        assert m % p == 0 and n % q == 0, "the super-entry shape must divide the last two modes"
        y = x.clone(memory_format=torch.contiguous_format)
        batch_shape = y.shape[:-2]
        options = {**options, "super": True}
        l, u = factors[-2].contiguous(), factors[-1].t().contiguous()
        if engine._sweep_super(y, l, u, batch_shape, options, quantizer_inputs, (p, q), inner_block_size, outer_block_size,
                               lead_factors=lead) is not None:
            return y
    # the explicit Kronecker row factor on the two-sided engines
    rows = x.numel() // x.size(-1)
    row_factor = functools.reduce(torch.kron, [f.contiguous() for f in factors[:-1]]) if len(factors) > 1 else torch.ones(1, 1, dtype=x.dtype, device=x.device)
    options = dict(sweep_options)
    if quantizer is not None:
        options["quantizer"] = quantizer
    run = engine.gptq_2d
    if tuple(super_entry_shape) != (1, 1):
        run, options["super_entry_shape"] = engine.gptq_2d_super_entry, tuple(super_entry_shape)
    z = run(x.reshape(rows, x.size(-1)), row_factor.contiguous(), factors[-1].t().contiguous(), quantizer_inputs=quantizer_inputs, **options)
    return z.reshape(x.shape)


@torch.no_grad()
def alg4(X: torch.Tensor, L, Q=None) -> torch.Tensor:
    """The reference's ``alg4(X, L, Q)`` by name and positional signature (gptq_2d_reference.py:269-294): ``L`` holds one
    unit lower triangular factor per mode, ``Q(values, *indices)`` rounds the entries of a stage given their index
    tensors (default: nearest integer).  Rounding runs on the mode-by-mode engine; any other ``Q`` is called stage by
    stage on the two-sided per-stage engine over the ``[n_1 ... n_{D-1}, n_D]`` view."""
    if Q is None:
        return gptq_d_sided(X, L)
    shape, n_last = X.shape, X.size(-1)

    def quantizer(y_flat, selection, *, out):
        flat = torch.arange(*selection.indices(y_flat.size(-1)), device=y_flat.device)
        indices = torch.unravel_index(flat, shape)
        out.copy_(Q(y_flat[..., selection], *indices))

    return gptq_d_sided(X, L, quantizer=quantizer, dense_row_factor=True)


@torch.no_grad()
def feedback_factors_from_grams(g: torch.Tensor, h: torch.Tensor, super_entry_shape: tuple[int, int] = (1, 1),
                                check: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """L from the output-side Gram ``g [m, m]`` and U from the input-side Gram ``h [n, n]`` (``U = ldl_of_inverse(h).T``),
    prepared together: both factorizations are chains of short dependent launches, so they advance block step by block
    step in the same launches (``g2d_ldl_of_inverse_pair``) and the pair costs little more than the larger one."""
    p, q = super_entry_shape
    assert g.dim() == 2 and g.size(0) == g.size(1) and h.dim() == 2 and h.size(0) == h.size(1), "expected square matrices"
    assert g.is_cuda and h.is_cuda and g.device == h.device, "the CUDA factor preparation requires CUDA tensors on one device"
    assert g.dtype == h.dtype, "both Grams must have the same dtype"
    m, n = g.size(0), h.size(0)
    assert p > 0 and q > 0 and m % p == 0 and n % q == 0, "the block sizes must divide the matrix sizes"
    if m == 0 or n == 0:
        return ldl_of_inverse(g, size=p, check=check), ldl_of_inverse(h, size=q, check=check).t()
    lib = _abi.library()
    code = _abi.dtype_code(g.dtype)
    works = [x.clone(memory_format=torch.contiguous_format) for x in (g, h)]  # the kernels factor in place
    outs = [torch.empty_like(w) for w in works]
    spaces = []
    for k in (m, n):
        need = ctypes.c_size_t()
        _abi.check(lib.g2d_ldl_workspace_bytes(code, k, ctypes.byref(need)), "g2d_ldl_workspace_bytes")
        spaces.append(torch.empty(need.value, dtype=torch.uint8, device=g.device))
    flags = torch.zeros(2, dtype=torch.int32, device=g.device)
    with torch.cuda.device(g.device):
        _abi.check(lib.g2d_ldl_of_inverse_pair(code, m, works[0].data_ptr(), p, outs[0].data_ptr(), spaces[0].data_ptr(), spaces[0].numel(),
                                               n, works[1].data_ptr(), q, outs[1].data_ptr(), spaces[1].data_ptr(), spaces[1].numel(),
                                               flags.data_ptr(), _abi.stream_of(g)), "g2d_ldl_of_inverse_pair")
    if check:
        _raise_for_flags(flags.tolist(), ("G", "H"))
    else:
        _PENDING.append((flags, ("G", "H")))
        if len(_PENDING) > _PENDING_LIMIT:  # a long unchecked run: settle the oldest call (it finished long ago)
            oldest, names = _PENDING.pop(0)
            _raise_for_flags(oldest.tolist(), names)
    return outs[0], outs[1].t()


_PENDING: list[tuple[torch.Tensor, tuple[str, ...]]] = []  # status flags of the calls made with check=False, oldest first
_PENDING_LIMIT = 256


def _raise_for_flags(pivots, names) -> None:
    for name, pivot in zip(names, pivots):
        if pivot < 0:
            raise RuntimeError("factor preparation: a bounded wait inside a tensor-core kernel ran out; the result is not valid")
        if pivot:
            raise torch.linalg.LinAlgError(f"factor preparation: {name} is not positive definite (pivot {pivot} is not positive)")


def last_flags() -> torch.Tensor | None:
    """The device-side ``int32`` status flags of the most recent unchecked factor preparation (G, H of a pair call),
    for callers that fold them into statistics of their own instead of raising."""
    return _PENDING[-1][0] if _PENDING else None


def check_pending() -> None:
    """Settle every ``feedback_factors_from_grams(..., check=False)`` call made so far: wait for them and raise what
    ``check=True`` would have raised (``torch.linalg.LinAlgError`` for a Gram that is not positive definite, as the
    reference's ``torch.linalg.cholesky`` does; ``RuntimeError`` for a bounded wait that ran out)."""
    while _PENDING:
        flags, names = _PENDING.pop(0)
        _raise_for_flags(flags.tolist(), names)
