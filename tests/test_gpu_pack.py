"""Packed codes on the GPU against the numpy restatement, and the round trip through the sweep's own output."""
import functools

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("m, n, bits, qmin", [(5, 13, 3, 0), (64, 200, 4, -8), (3, 1024, 2, -2), (17, 96, 8, -128), (9, 40, 5, 0), (1, 7, 1, 0)])
def test_pack_matches_oracle(oracle, dtype, m, n, bits, qmin):
    import packed_codes as P

    rng = np.random.default_rng(m * n + bits)
    scale = (0.01 + rng.random((m, n))).astype(dtype)
    zero = np.rint(rng.uniform(qmin, qmin + 2 ** bits - 1, (m, n))).astype(dtype)
    codes = rng.integers(qmin - 2, qmin + 2 ** bits + 2, (m, n))  # some outside the field: they must clamp
    z = ((codes - zero) * scale).astype(dtype)
    expected = oracle.pack_codes(z, scale, zero, qmin, bits)
    cuda = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    packed = P.pack_codes(cuda(z), cuda(scale), cuda(zero), qmin=qmin, bits=bits)
    assert packed.shape == expected.shape and np.array_equal(packed.cpu().numpy(), expected)
    back = P.unpack_codes(packed, cuda(scale), cuda(zero), qmin=qmin, bits=bits, n=n, dtype=torch.from_numpy(z).dtype)
    assert np.array_equal(back.cpu().numpy(), oracle.unpack_codes(expected, scale, zero, qmin, bits, n, dtype))
    # per-row scales and a scalar zero point, passed as broadcastable tensors
    row_scale = scale[:, :1].copy()
    z_rows = ((np.clip(codes, qmin, qmin + 2 ** bits - 1)) * row_scale).astype(dtype)
    packed = P.pack_codes(cuda(z_rows), cuda(row_scale), torch.zeros((), device="cuda"), qmin=qmin, bits=bits)
    assert np.array_equal(packed.cpu().numpy(), oracle.pack_codes(z_rows, row_scale, 0.0, qmin, bits))
    back = P.unpack_codes(packed, cuda(row_scale), torch.zeros((), device="cuda"), qmin=qmin, bits=bits, n=n, dtype=torch.from_numpy(z).dtype)
    assert torch.equal(back, cuda(z_rows))


def test_sweep_output_round_trips():
    """The sweep's dequantised result is exactly recovered from its packed codes (INT4 per-row scales, INT3 groups with zero points)."""
    import gptq_2d as G
    import packed_codes as P
    import quantizer_int as Q

    gen = torch.Generator(device="cuda").manual_seed(5)
    m, n = 384, 512
    w = 0.02 * torch.randn(m, n, generator=gen, device="cuda")
    l = torch.tril(torch.randn(m, m, generator=gen, device="cuda") * (0.3 / m ** .5), -1)
    u = torch.triu(torch.randn(n, n, generator=gen, device="cuda") * (0.3 / n ** .5), 1)
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16)
    zero = torch.zeros(1, 1, device="cuda")
    z = G.gptq_2d(w, l, u, quantizer=functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7),
                  quantizer_inputs=(scale.expand(m, n), zero.expand(m, n)))
    packed = P.pack_codes(z, scale, zero, qmin=-8, bits=4)
    assert packed.shape == (m, n // 2)
    assert torch.equal(P.unpack_codes(packed, scale, zero, qmin=-8, bits=4, n=n), z)
    groups = w.view(m, n // 128, 128)
    lo, hi = groups.amin(-1), groups.amax(-1)
    scale3 = ((hi - lo) / 7).repeat_interleave(128, dim=1).contiguous()
    zero3 = torch.round(-lo / ((hi - lo) / 7)).repeat_interleave(128, dim=1).contiguous()
    z3 = G.gptq_2d(w, l, u, quantizer=functools.partial(Q.affine_quantizer_triton, qmin=0, qmax=7), quantizer_inputs=(scale3, zero3))
    packed3 = P.pack_codes(z3, scale3, zero3, qmin=0, bits=3)
    assert packed3.shape == (m, n * 3 // 8)
    assert torch.equal(P.unpack_codes(packed3, scale3, zero3, qmin=0, bits=3, n=n), z3)
    assert P.pack_codes(z[:0], scale[:0], zero, qmin=-8, bits=4).shape == (0, n // 2)
