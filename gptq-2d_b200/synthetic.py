"""Seeded synthetic layers with the shapes and value distributions of the benchmark configurations.

The reference ships no weights, Hessians or calibration data, so every measurement uses these stand-ins:
weights ``W = sigma_w * randn(m, n)`` (optionally with a fraction of 10-sigma outliers) and, for each side, a
Hessian factor ``H = X^T X / k + lambda I`` built from activations ``X = randn(k, dim) * exp(sigma_h * randn(dim))``
(log-normal per-channel scales) with ``lambda = damp * mean(diag(X^T X / k))``.  ``G`` (m x m) belongs to the
output side and gives L; ``H`` (n x n) belongs to the input side and gives U.
"""
from __future__ import annotations

import torch


def hessian_factor(dim: int, samples: int, sigma_h: float, damp: float, generator: torch.Generator,
                   device, dtype=torch.float32, chunk: int = 4096) -> torch.Tensor:
    """``X^T X / samples + lambda I`` for seeded heavy-tailed activations, accumulated in row chunks."""
    channel = torch.exp(sigma_h * torch.randn(dim, generator=generator, device=device, dtype=dtype))
    h = torch.zeros(dim, dim, device=device, dtype=dtype)
    on_tensor_cores = h.is_cuda and dtype == torch.float32 and dim % 4 == 0  # the library's own accumulation kernel
    done = 0
    while done < samples:
        rows = min(chunk, samples - done)
        x = torch.randn(rows, dim, generator=generator, device=device, dtype=dtype) * channel
        if on_tensor_cores:
            import kron_factors

            kron_factors.accumulate_gram(h, x, 1.0 / samples)
        else:
            h.addmm_(x.T, x, alpha=1.0 / samples)
        done += rows
    h.diagonal().add_(damp * h.diagonal().mean())
    return h


def make_layer(m: int, n: int, seed: int, device, *, sigma_w: float = 0.02, sigma_h: float = 1.0, damp: float = 0.01,
               samples: int = 8192, outliers: float = 0.0, dtype=torch.float32, input_seed: int | None = None,
               without_input_factor: bool = False):
    """Return ``(W [m, n], G [m, m], H [n, n])`` for one seeded synthetic layer.

    Matrices that read the same activations (the q, k, v projections of a block; gate and up) share their input-side
    factor: give them the same ``input_seed``, which then seeds H alone (``shared_input_factor`` makes just that
    matrix); ``without_input_factor`` returns None in its place."""
    generator = torch.Generator(device=device).manual_seed(seed)
    w = sigma_w * torch.randn(m, n, generator=generator, device=device, dtype=dtype)
    if outliers > 0:
        mask = torch.rand(m, n, generator=generator, device=device) < outliers
        signs = torch.where(torch.rand(m, n, generator=generator, device=device) < 0.5, -1.0, 1.0).to(dtype)
        w = torch.where(mask, 10 * sigma_w * signs, w)
    g = hessian_factor(m, samples, sigma_h, damp, generator, device, dtype)
    if without_input_factor:
        return w, g, None
    if input_seed is not None:
        return w, g, shared_input_factor(n, input_seed, device, sigma_h=sigma_h, damp=damp, samples=samples, dtype=dtype)
    h = hessian_factor(n, samples, sigma_h, damp, generator, device, dtype)
    return w, g, h


def shared_input_factor(n: int, input_seed: int, device, *, sigma_h: float = 1.0, damp: float = 0.01, samples: int = 8192,
                        dtype=torch.float32) -> torch.Tensor:
    """The input-side factor ``H [n, n]`` that every matrix with this ``input_seed`` uses."""
    generator = torch.Generator(device=device).manual_seed(input_seed)
    return hessian_factor(n, samples, sigma_h, damp, generator, device, dtype)


def objective(z: torch.Tensor, x: torch.Tensor, g: torch.Tensor, h: torch.Tensor) -> float:
    """The two-sided objective ``tr((Z - X)^T G (Z - X) H)`` in float64."""
    r = (z - x).double()
    return ((g.double() @ r) * (r @ h.double())).sum().item()
