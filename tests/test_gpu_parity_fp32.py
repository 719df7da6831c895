"""float32 parity of the fused engine and of the factor preparation on the benchmark's own distributions.

The second benchmark configuration draws weights with 0.1 % outliers at 10 sigma and Hessian factors with log-normal
(sigma = 1) channel scales; its feedback factors are far from the benign random triangles of the smaller tests.
Free-running float32 trajectories of this algorithm are chaotic (two float32 implementations of the reference
disagree with each other on percents of the codes at n >= 1024), so parity is measured under teacher forcing: the
rounding decisions of the oracle's float64 run are imposed on the engine, which reports the value every entry had at
the moment it would have been rounded.  The bar: the would-be codes equal the oracle's on >= 99.9 % of the entries and
every mismatch lies within TIE_WINDOW code units of a rounding tie.  The oracle's own float32 run (the restated
reference path in float32) goes through the same measurement, and the figures of both are written down side by side
when G2D_REPORT_DIR names a directory.

Factors come from the oracle's float64 ``ldl_of_inverse`` (LAPACK, as the reference computes them), not from the
library under test.
"""
import functools
import json
import os

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu

TIE_WINDOW = 1e-5        # code units: the bar the project states for float32
MAX_DEVIATION = 2e-4     # code units: largest |y_pre - exact| accepted (the reference's own float32: about 1e-4)

_CASES: dict = {}
_REPORT: dict = {}


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _report(name, values):
    _REPORT[name] = values
    directory = os.environ.get("G2D_REPORT_DIR")
    if directory:
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "parity_fp32.json"), "w") as f:
            json.dump(_REPORT, f, indent=1, sort_keys=True)


def config1_case(oracle, m, n):
    """Inputs, the float64 decisions and the exact pre-rounding values of one seeded layer (computed once per size)."""
    if (m, n) not in _CASES:
        w, g, h = oracle.config1_layer(m, n, seed=m + n)
        l = oracle.ldl_of_inverse_lapack(g.astype(np.float64)).astype(np.float32)
        u = np.ascontiguousarray(oracle.ldl_of_inverse_lapack(h.astype(np.float64)).T).astype(np.float32)
        l, u = np.tril(l, -1), np.triu(u, 1)
        scale = np.ascontiguousarray(np.broadcast_to(oracle.absmax_scale(w, -8, 7, oracle.FP16), (m, n)))
        zero = np.zeros((m, n), dtype=np.float32)
        as64 = lambda a: a.astype(np.float64)
        z_star = oracle.sweep(as64(w), as64(l), as64(u), kind=oracle.Q_AFFINE, scale=as64(scale), zero_point=as64(zero), qmin=-8, qmax=7)
        z32 = z_star.astype(np.float32)  # code * fp16 scale: exact in float32
        assert np.array_equal(z32.astype(np.float64), z_star)
        _, exact = oracle.sweep(as64(w), as64(l), as64(u), kind=oracle.Q_FORCED, forced_z=z_star, return_y_pre=True)
        _, ref32 = oracle.sweep(w, l, u, kind=oracle.Q_FORCED, forced_z=z32, return_y_pre=True)
        _CASES[(m, n)] = dict(w=w, g=g, h=h, l=l, u=u, scale=scale, zero=zero, z=z32, exact=exact, ref32=ref32)
    return _CASES[(m, n)]


def tie_statistics(y_pre, case):
    """Deviation from the exact pre-rounding values and the would-be mismatches, in code units."""
    scale = case["scale"].astype(np.float64)
    t = y_pre.astype(np.float64) / scale
    deviation = np.abs(t - case["exact"] / scale)
    codes = np.rint(case["z"].astype(np.float64) / scale)
    mismatch = np.clip(np.rint(t), -8, 7) != codes
    to_tie = np.abs(np.abs(t - np.floor(t)) - 0.5)
    return {
        "entries": int(t.size), "mismatches": int(mismatch.sum()), "mismatch_fraction": float(mismatch.mean()),
        "worst_mismatch_to_tie": float(to_tie[mismatch].max()) if mismatch.any() else 0.0,
        "mismatches_beyond_1e-5": int((to_tie[mismatch] > 1e-5).sum()),
        "deviation_median": float(np.median(deviation)), "deviation_p99": float(np.quantile(deviation, 0.99)),
        "deviation_max": float(deviation.max()),
        "l_max": float(np.abs(case["l"]).max()), "u_max": float(np.abs(case["u"]).max()),
    }


@pytest.fixture(params=[1, 2, 3], ids=["tile-schedule", "macro-schedule", "pipelined-schedule"])
def schedule(request):
    import gptq_2d as G

    before = G.SWEEP_SCHEDULE
    G.SWEEP_SCHEDULE = request.param
    yield request.param
    G.SWEEP_SCHEDULE = before


def forced_check(oracle, m, n, label):
    import gptq_2d as G

    case = config1_case(oracle, m, n)
    z, y_pre = G.gptq_2d_forced(cuda(case["w"]), cuda(case["l"]), cuda(case["u"]), cuda(case["z"]))
    G.check_status()
    assert torch.equal(z.cpu(), torch.from_numpy(case["z"]))
    ours, reference = tie_statistics(y_pre.cpu().numpy(), case), tie_statistics(case["ref32"], case)
    _report(f"{m}x{n} {label}", {"engine": ours, "oracle_float32": reference})
    assert ours["mismatch_fraction"] <= 1e-3, ours
    assert ours["worst_mismatch_to_tie"] <= TIE_WINDOW, (ours, reference)
    assert ours["deviation_max"] <= MAX_DEVIATION, (ours, reference)
    return ours, reference


def test_teacher_forced_config1_2048(oracle, schedule):
    """2048 x 2048 under every launch schedule: the macro and the pipelined schedule run their far update several times."""
    forced_check(oracle, 2048, 2048, ("tile", "macro", "pipelined")[schedule - 1])


def test_teacher_forced_config1_4096_pipelined(oracle):
    """The configuration's full size on the default (pipelined, tensor-core) schedule."""
    forced_check(oracle, 4096, 4096, "default")


def test_free_run_config1_mismatches_lie_at_ties(oracle):
    """A free float32 run: every entry is the quantizer applied to the engine's own pre-rounding value (so no code is
    ever wrong by more than the engine's deviation), and against the float64 oracle the objective stays within the
    spread the float32 oracle itself shows on the same inputs."""
    import _abi
    import gptq_2d as G

    m = n = 2048
    case = config1_case(oracle, m, n)
    w, l, u, scale, zero = (cuda(case[k]) for k in ("w", "l", "u", "scale", "zero"))
    y, _, _, batch_shape = G._prepare_output(w, l, u, False)
    y_pre = torch.empty_like(y)
    G._sweep_fused(y, l, u, batch_shape, dict(kind=_abi.Q_AFFINE, qmin=-8, qmax=7), (scale, zero), y_pre=y_pre)
    G.check_status()
    assert torch.equal(y, torch.clamp(torch.round(y_pre / scale), -8, 7) * scale)
    free32 = oracle.sweep(case["w"], case["l"], case["u"], kind=oracle.Q_AFFINE, scale=case["scale"], zero_point=case["zero"], qmin=-8, qmax=7)
    g, h = case["g"], case["h"]
    exact_objective = oracle.objective(case["z"], case["w"], g, h)
    ours = oracle.objective(y.cpu().numpy(), case["w"], g, h) / exact_objective - 1
    reference = oracle.objective(free32, case["w"], g, h) / exact_objective - 1
    agree = float((torch.round(y / scale).cpu().numpy() == np.rint(case["z"] / case["scale"])).mean())
    agree_reference = float((np.rint(free32 / case["scale"]) == np.rint(case["z"] / case["scale"])).mean())
    _report("2048x2048 free run", {"objective_rel_engine": ours, "objective_rel_oracle_float32": reference,
                                   "codes_equal_engine": agree, "codes_equal_oracle_float32": agree_reference})
    assert abs(ours) <= max(1e-4, 3 * abs(reference))


def test_quotient_by_reciprocal_flips_no_code():
    """Inside the fused float32 sweep the affine quantizer divides by a Newton-refined reciprocal with one residual
    correction instead of an IEEE division.  On random values and on values placed at and next to rounding ties, with
    fp16-valued scales as the INT4 configurations use, the fused path (one tile, no feedback: L = U = 0) must return what
    the stand-alone quantizer kernel (IEEE division) returns; the number of differing entries is written down."""
    import gptq_2d as G
    import quantizer_int as Q

    gen = torch.Generator(device="cuda").manual_seed(5)
    m, n = 512, 512
    scale = (torch.rand(m, 1, generator=gen, device="cuda") * 0.02 + 1e-4).half().float().expand(m, n).contiguous()
    codes = torch.randint(-9, 9, (m, n), generator=gen, device="cuda").float()
    offsets = torch.tensor([0.5, 0.5 - 1e-6, 0.5 + 1e-6, 0.25, 0.4999999, 0.0], device="cuda")
    y = (codes + offsets[torch.randint(0, 6, (m, n), generator=gen, device="cuda")]) * scale
    y[::2] = torch.randn(m // 2, n, generator=gen, device="cuda") * 0.05
    zero = torch.zeros(m, n, device="cuda")
    l, u = torch.zeros(m, m, device="cuda"), torch.zeros(n, n, device="cuda")
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7)
    fused = G.gptq_2d(y, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
    plain = torch.empty_like(y)
    for s in range(m + n - 1):  # the stand-alone kernel, one anti-diagonal at a time as the generic engine calls it
        selection = G._antidiagonal_slices(m=m, n=n, s=s)[2]
        out = torch.empty(len(range(*selection.indices(m * n))), device="cuda")
        quantizer(y.flatten(), selection, scale, zero, out=out)
        plain.flatten()[selection] = out
    differing = int((fused != plain).sum().item())
    _report("reciprocal division", {"entries": m * n, "differing": differing})
    assert differing == 0


def test_float32_factors_golden_large():
    """The tensor-core factor preparation against the reference's float32 and float64 factors of heavy-tailed Grams
    (n = 1024, 2048, condition number about 1.3e4).  Distance to the float64 factor, largest entry over the stored rows:
    the reference's float32 LAPACK result 1.1e-6 / 0.8e-6, torch's float32 CUDA path on a B200 1.7e-6, this library
    3.6e-6 / 3.4e-6 (measured); the bound is 6e-6, four times the reference's own float32 distance over the whole factor."""
    import kron_factors as K
    from oracle import oracle

    g = load_golden("factors_fp32_large.npz")
    report = {}
    for n in (1024, 2048):
        gram = cuda(oracle.dyadic_gram(n, seed=n))
        rows = g[f"rows{n}"]
        single = K.ldl_of_inverse(gram)
        l_pair, u_pair = K.feedback_factors_from_grams(gram, gram, check=True)
        assert torch.equal(single, l_pair) and torch.equal(u_pair.T, l_pair)
        ours = single.double().cpu().numpy()[rows]
        gap = float(np.abs(ours - g[f"l64_{n}"]).max())
        reference_gap = float(np.abs(g[f"l32_{n}"].astype(np.float64) - g[f"l64_{n}"]).max())
        report[str(n)] = {"engine_vs_float64": gap, "reference_float32_vs_float64": reference_gap, "whole_factor_reference_gap": float(g[f"gap{n}"]),
                          "l_max": float(g[f"lmax{n}"])}
        _report("factors golden", report)
        assert gap <= 6e-6 and gap <= 8 * float(g[f"gap{n}"]), report


def test_float32_factors_4096(oracle):
    """n = 4096, sigma_h = 1: the pair path (the one the benchmark times) against the oracle's float64 factor.  Measured
    4.8e-6 (a float32 LAPACK factorization of the same matrix: 1.6e-6, torch's float32 CUDA path: 2.3e-6); the bound does
    not grow with n, because the long sums are cut into slices that are added up in round-to-nearest arithmetic."""
    import kron_factors as K

    n = 4096
    gram_g, gram_h = oracle.dyadic_gram(n, seed=7), oracle.dyadic_gram(n, seed=8)
    l, u = K.feedback_factors_from_grams(cuda(gram_g), cuda(gram_h), check=True)
    report = {}
    for name, ours, gram in (("L", l, gram_g), ("U^T", u.T, gram_h)):
        exact = oracle.ldl_of_inverse_lapack(gram.astype(np.float64))
        gap = float(np.abs(ours.double().cpu().numpy() - exact).max())
        report[name] = {"engine_vs_float64": gap, "l_max": float(np.abs(exact).max())}
        _report("factors 4096", report)
        assert gap <= 8e-6, report
