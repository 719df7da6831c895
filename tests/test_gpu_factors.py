"""GPU tests of the factor preparation.  The reference computes these factors with LAPACK / cuSOLVER through
torch.linalg, so parity is to a tolerance (stated per case) plus the defining properties."""
import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    import kron_factors
    return kron_factors


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check_structure(l, size):
    n = l.size(0)
    block = torch.arange(n, device=l.device) // size
    same = block[:, None] == block[None, :]
    assert torch.equal(l[same], torch.eye(n, dtype=l.dtype, device=l.device)[same])  # identity diagonal blocks, exactly
    assert (l[block[:, None] < block[None, :]] == 0).all()


def test_golden_factors(K):
    g = load_golden("factors.npz")
    for n in (1, 7, 64, 200):
        m = cuda(g[f"g{n}"])
        before = m.clone()
        l = K.ldl_of_inverse(m)
        assert torch.equal(m, before)  # the input is left alone
        assert torch.allclose(l.cpu(), torch.from_numpy(g[f"l{n}"]), rtol=0, atol=1e-9)
        check_structure(l, 1)
    for size in (1, 2, 4, 16):
        l = K.ldl_of_inverse(cuda(g["g48"]), size)
        assert torch.allclose(l.cpu(), torch.from_numpy(g[f"l48_{size}"]), rtol=0, atol=1e-9)
        check_structure(l, size)
    l = K.ldl_of_inverse(cuda(g["g256_f32"]))
    assert (l.cpu() - torch.from_numpy(g["l256_f32"])).abs().max() < 5e-5


@pytest.mark.parametrize("n,size", [(130, 1), (130, 5), (1000, 1), (960, 16), (1536, 3)])
def test_against_oracle_and_properties(K, oracle, n, size):
    rng = np.random.default_rng(n + size)
    x = rng.standard_normal((2 * n, n)) * np.exp(0.5 * rng.standard_normal(n))
    gram = x.T @ x / (2 * n)
    gram += 0.01 * np.mean(np.diag(gram)) * np.eye(n)
    l = K.ldl_of_inverse(cuda(gram), size)
    if n <= 1000:
        assert np.abs(l.cpu().numpy() - oracle.ldl_of_inverse(gram, size)).max() < 1e-8
    check_structure(l, size)
    # G^{-1} = L Lambda L^T  <=>  L^T G L is block diagonal
    d = l.T @ cuda(gram) @ l
    block = torch.arange(n, device="cuda") // size
    off = d[block[:, None] != block[None, :]]
    assert off.abs().max().item() < 1e-9 * d.diagonal().abs().max().item()
    # float32 stays close to the float64 factor
    l32 = K.ldl_of_inverse(cuda(gram.astype(np.float32)), size)
    assert (l32.double() - l).abs().max().item() < 2e-3
    check_structure(l32, size)


def test_feedback_factors_and_errors(K):
    gen = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(24, 24, generator=gen, device="cuda", dtype=torch.float64)
    b = torch.randn(40, 40, generator=gen, device="cuda", dtype=torch.float64)
    l, u = K.feedback_factors(a, b, (4, 8))
    check_structure(l, 4)
    check_structure(u.T, 8)
    from gptq_2d_reference import ldl_of_inverse
    assert torch.equal(ldl_of_inverse(a.T @ a, size=4), l)
    with pytest.raises(torch.linalg.LinAlgError):
        K.ldl_of_inverse(-torch.eye(70, device="cuda", dtype=torch.float64))
    assert K.ldl_of_inverse(torch.empty(0, 0, device="cuda")).shape == (0, 0)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("m, n, p, q", [(200, 330, 1, 1), (1100, 256, 2, 4), (64, 1345, 1, 5), (640, 640, 1, 1)])
def test_pair_equals_two_single_calls(K, dtype, m, n, p, q):
    """Both factors of a layer prepared in shared launches are bit-identical to one call per factor, whatever the sizes."""
    gen = torch.Generator(device="cuda").manual_seed(m + n)
    grams = []
    for k in (m, n):
        a = torch.randn(k + 32, k, generator=gen, device="cuda", dtype=dtype)
        grams.append(a.T @ a / k + 0.01 * torch.eye(k, device="cuda", dtype=dtype))
    l, u = K.feedback_factors_from_grams(grams[0], grams[1], (p, q), check=True)
    assert torch.equal(l, K.ldl_of_inverse(grams[0], p))
    assert torch.equal(u, K.ldl_of_inverse(grams[1], q).T)
    check_structure(l, p)
    check_structure(u.T, q)


def test_pair_reports_the_failing_factor(K):
    good = torch.eye(130, device="cuda", dtype=torch.float64)
    with pytest.raises(torch.linalg.LinAlgError, match="H is not positive definite"):
        K.feedback_factors_from_grams(good, -torch.eye(70, device="cuda", dtype=torch.float64), check=True)
    with pytest.raises(torch.linalg.LinAlgError, match="G is not positive definite"):
        K.feedback_factors_from_grams(-good, torch.eye(70, device="cuda", dtype=torch.float64), check=True)


def test_d_sided_golden(K):
    """gptq_2d_reference.py:450-478: N-factor rounding equals Algorithm 1 on the explicit Kronecker Gram (values from the reference's alg4)."""
    g = load_golden("d_sided_fp64.npz")
    for k in range(int(g["count"])):
        x = cuda(g[f"x{k}"])
        factors = [cuda(g[f"l{k}_{d}"]) for d in range(x.dim())]
        z = K.gptq_d_sided(x, factors)
        assert torch.equal(z.cpu(), torch.from_numpy(g[f"z{k}"])), k


@pytest.mark.parametrize("k, n", [(1000, 512), (37, 132), (4096, 1100), (64, 4)])
def test_gram_accumulation(K, k, n):
    """h += alpha x^T x on the tensor cores stays at float32 fidelity (3xTF32) and is symmetric bit for bit."""
    gen = torch.Generator(device="cuda").manual_seed(k + n)
    x = torch.randn(k, n, generator=gen, device="cuda") * torch.exp(torch.randn(n, generator=gen, device="cuda"))
    h0 = torch.randn(n, n, generator=gen, device="cuda")
    h0 = h0 + h0.T
    h = K.accumulate_gram(h0.clone(), x, alpha=1.0 / k)
    want = h0.double() + x.double().T @ x.double() / k
    scale = want.abs().max().item()
    assert (h.double() - want).abs().max().item() <= 3e-6 * scale
    assert torch.equal(h, h.T)
    again = K.accumulate_gram(h0.clone(), x, alpha=1.0 / k)
    assert torch.equal(h, again)  # one owner per entry: run-to-run identical
