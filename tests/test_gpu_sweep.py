"""GPU parity tests of the sweep engines against the CPU oracle and the golden vectors.

Every call goes through the package's public API, which reaches the kernels only through the C ABI.
fp64 results must be bit-identical (the reference's own standard, test_gptq_2d.py:89); fp32 follows
the project's stated bar: objective within 1e-4 relative, codes equal on >= 99.9 % of entries, and under
teacher-forced replay every would-be mismatch within 1e-5 code units of a rounding tie.
"""
import functools

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu

BLOCKS = ((0, 0), (1, 0), (2, 8), (3, 11))  # test_gptq_2d.py:81


@pytest.fixture(scope="module")
def api():
    import gptq_2d
    import quantizer_int
    return gptq_2d, quantizer_int


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def python_round(y_flat, selection, *, out):
    """A quantizer the package cannot recognise: forces the generic engine."""
    selected = selection(y_flat) if callable(selection) else y_flat[..., selection]
    torch.round(selected, out=out)


@pytest.fixture(params=[1, 2, 3], ids=["tile-schedule", "macro-schedule", "pipelined-schedule"])
def schedule(request, api):
    """Run a test under every launch schedule of the fused engine."""
    G, _ = api
    before = G.SWEEP_SCHEDULE
    G.SWEEP_SCHEDULE = request.param
    yield request.param
    G.SWEEP_SCHEDULE = before


def test_fused_round_fp64_golden(api, schedule):
    G, _ = api
    g = load_golden("sweep_fp64.npz")
    for k, (m, n, p, q) in enumerate(g["cases"]):
        if (p, q) != (1, 1):
            continue
        x, l, u = cuda(g[f"x{k}"]), cuda(g[f"l{k}"]), cuda(g[f"u{k}"])
        z = G.gptq_2d(x, l, u)
        assert torch.equal(z.cpu(), torch.from_numpy(g[f"z_round{k}"])), (m, n)
        assert torch.equal(x.cpu(), torch.from_numpy(g[f"x{k}"]))  # out of place leaves X alone
        z1 = G.gptq_2d_super_entry(x, l, u, super_entry_shape=(1, 1))
        assert torch.equal(z1, z)


def test_generic_engine_fp64_golden(api):
    G, Q = api
    g = load_golden("sweep_fp64.npz")
    for k, (m, n, p, q) in enumerate(g["cases"]):
        x, l, u = cuda(g[f"x{k}"]), cuda(g[f"l{k}"]), cuda(g[f"u{k}"])
        expected = torch.from_numpy(g[f"z_round{k}"])
        expected_absmax = torch.from_numpy(g[f"z_absmax{k}"])
        joint = functools.partial(Q.int_abs_max_quantizer_cuda, qmin=-2, qmax=1, dtype=torch.bfloat16)
        for inner, outer in BLOCKS:
            z = G.gptq_2d_super_entry(x, l, u, quantizer=python_round, super_entry_shape=(int(p), int(q)),
                                      inner_block_size=inner, outer_block_size=outer)
            assert torch.equal(z.cpu(), expected), (m, n, p, q, inner, outer)
            z = G.gptq_2d_super_entry(x, l, u, quantizer=joint, super_entry_shape=(int(p), int(q)),
                                      inner_block_size=inner, outer_block_size=outer)
            assert torch.equal(z.cpu(), expected_absmax), ("absmax", m, n, p, q, inner, outer)
            if (p, q) == (1, 1):
                z = G.gptq_2d(x, l, u, quantizer=python_round, inner_block_size=inner, outer_block_size=outer)
                assert torch.equal(z.cpu(), expected), (m, n, inner, outer)
        z = G.gptq_2d_super_entry_torch(x, l, u, quantizer=python_round, super_entry_shape=(int(p), int(q)))
        assert torch.equal(z.cpu(), expected)


def test_default_blocks_medium_fp64(api, oracle, schedule):
    """Default block sizes (32 / 512 and 8 / 64) on a size that flushes at both levels."""
    G, _ = api
    rng = np.random.default_rng(5)
    m, n = 150, 700
    x = 4 * rng.standard_normal((m, n))
    l, u = np.tril(.05 * rng.standard_normal((m, m)), -1), np.triu(.05 * rng.standard_normal((n, n)), 1)
    expected = torch.from_numpy(oracle.sweep(x, l, u))
    xc, lc, uc = cuda(x), cuda(l), cuda(u)
    assert torch.equal(G.gptq_2d(xc, lc, uc, quantizer=python_round).cpu(), expected)
    assert torch.equal(G.gptq_2d(xc, lc, uc).cpu(), expected)
    expected = torch.from_numpy(oracle.sweep(x, l, u, super_entry_shape=(2, 5)))
    z = G.gptq_2d_super_entry(xc, lc, uc, quantizer=python_round, super_entry_shape=(2, 5))
    assert torch.equal(z.cpu(), expected)


def test_batches_inplace_and_quantizer_inputs(api, schedule):
    """test_gptq_2d.py:129-147: broadcast batches, per-entry scales, in and out of place, both engines."""
    G, Q = api
    g = load_golden("sweep_batched_fp64.npz")

    def round_to_scale(y_flat, selection, scale, *, out):
        torch.div(y_flat[..., selection], scale.flatten(start_dim=-2)[..., selection], out=out).round_().mul_(scale.flatten(start_dim=-2)[..., selection])

    for k in range(int(g["count"])):
        x, l, u, scale = cuda(g[f"x{k}"]), cuda(g[f"l{k}"]), cuda(g[f"u{k}"]), cuda(g[f"scale{k}"])
        expected = torch.from_numpy(g[f"z{k}"])
        zero = torch.zeros(1, 1, device="cuda", dtype=torch.float64).expand(x.shape[-2:])
        before = x.clone()
        z = G.gptq_2d(x, l, u, quantizer=Q.affine_quantizer_triton, quantizer_inputs=(scale, zero))
        assert z.shape == expected.shape and torch.equal(z.cpu(), expected)
        z = G.gptq_2d(x, l, u, quantizer=round_to_scale, quantizer_inputs=(scale,), inner_block_size=3, outer_block_size=7)
        assert torch.equal(z.cpu(), expected)
        for quantizer, inputs in ((Q.affine_quantizer_torch, (scale, zero)), (round_to_scale, (scale,))):
            target = x.expand(*expected.shape).clone()
            result = G.gptq_2d(target, l, u, quantizer=quantizer, quantizer_inputs=inputs, inplace=True)
            assert result.data_ptr() == target.data_ptr() and torch.equal(result.cpu(), expected)
        assert torch.equal(x, before)


def test_quartic_reference_64(api):
    G, Q = api
    g = load_golden("quartic_64_fp64.npz")
    x, l, u, scale = cuda(g["x"]), cuda(g["l"]), cuda(g["u"]), cuda(g["scale"])
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=float(g["qmin"]), qmax=float(g["qmax"]))
    z = G.gptq_2d(x, l, u, quantizer=quantizer, quantizer_inputs=(scale, torch.zeros_like(scale)))
    assert torch.equal(z.cpu(), torch.from_numpy(g["z"]))


def _objective(z, x, g, h):
    r = (z - x).double()
    return ((g.double() @ r) * (r @ h.double())).sum().item()


def test_config0_fp32(api, schedule):
    """The first benchmark configuration (256 x 256 fp32 INT4, fp16 row scales) and its 64 x 64 companion."""
    G, Q = api
    for n in (64, 256):
        g = load_golden(f"config0_{n}_fp32.npz")
        w, l, u = cuda(g["w"]), cuda(g["l"]), cuda(g["u"])
        scale = cuda(g["scale"]).expand(n, n)  # stride (1, 0): per-row scales are not materialised
        zero = torch.zeros(1, 1, device="cuda").expand(n, n)
        quantizer = functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7)
        z = G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
        expected = cuda(g["z"])
        codes, expected_codes = torch.round(z / scale), torch.round(expected / scale)
        assert codes.min() >= -8 and codes.max() <= 7
        assert (codes == expected_codes).double().mean().item() >= 0.999
        gm, hm = cuda(g["g"]), cuda(g["h"])
        assert abs(_objective(z, w, gm, hm) / _objective(expected, w, gm, hm) - 1) <= 1e-4
        # the generic engine with the same quantizer called per stage
        z2 = G.gptq_2d(w, l, u, quantizer=lambda *a, **k: quantizer(*a, **k), quantizer_inputs=(scale.contiguous(), zero.contiguous()))
        assert (torch.round(z2 / scale) == expected_codes).double().mean().item() >= 0.999


@pytest.mark.parametrize("m,n", [(256, 256), (1024, 1024), (320, 1100), (196, 332)])
def test_teacher_forced_fp32(api, oracle, m, n, schedule):
    """Teacher-forced parity at fp32: with the rounding decisions imposed from the oracle's run, the engine's
    pre-rounding values must lead to the same codes except within 1e-5 code units of a tie."""
    G, Q = api
    rng = np.random.default_rng(m + n)
    w = (0.02 * rng.standard_normal((m, n))).astype(np.float32)
    l = np.tril(rng.standard_normal((m, m)) * (0.3 / np.sqrt(m)), -1).astype(np.float32)
    u = np.triu(rng.standard_normal((n, n)) * (0.3 / np.sqrt(n)), 1).astype(np.float32)
    scale = oracle.absmax_scale(w, -8, 7, oracle.FP16)
    full, zero = np.broadcast_to(scale, (m, n)), np.zeros((m, n), dtype=np.float32)
    z_star = oracle.sweep(w.astype(np.float64), l.astype(np.float64), u.astype(np.float64), kind=oracle.Q_AFFINE,
                          scale=full.astype(np.float64), zero_point=zero.astype(np.float64), qmin=-8, qmax=7)
    z, y_pre = G.gptq_2d_forced(cuda(w), cuda(l), cuda(u), cuda(z_star.astype(np.float32)))
    assert torch.equal(z.cpu(), torch.from_numpy(z_star.astype(np.float32)))
    _, y_pre_oracle = oracle.sweep(w, l, u, kind=oracle.Q_FORCED, forced_z=z_star.astype(np.float32), return_y_pre=True)
    y_pre = y_pre.cpu().numpy()
    units = np.abs(y_pre.astype(np.float64) - y_pre_oracle.astype(np.float64)) / full
    assert units.max() < 2e-4, units.max()
    would_be = np.clip(np.rint(y_pre.astype(np.float64) / full), -8, 7)
    star = np.rint(z_star / full)
    mismatch = would_be != star
    assert mismatch.mean() <= 1e-3
    t = y_pre.astype(np.float64) / full
    distance_to_tie = np.abs(np.abs(t - np.floor(t)) - 0.5)
    assert (distance_to_tie[mismatch] <= 1e-5).all()


@pytest.mark.parametrize("m,n", [(2048, 3072), (1000, 1356)])
def test_self_consistency_large_fp32(api, schedule, m, n):
    """Size-independent properties on a larger free run: Z is the quantizer applied to the engine's own
    pre-rounding values, and Z - X = L E U with E = Z - Y_pre (the defining identity of the sweep).  The second shape
    ends in ragged tiles in both directions (multiples of 4, so every schedule takes it): the parameters of entries
    outside the matrix and the feedback pushed to ragged neighbour tiles."""
    import _abi
    G, Q = api
    gen = torch.Generator(device="cuda").manual_seed(1)
    w = 0.02 * torch.randn(m, n, generator=gen, device="cuda")
    l = torch.tril(torch.randn(m, m, generator=gen, device="cuda") * (0.3 / m ** .5), -1)
    u = torch.triu(torch.randn(n, n, generator=gen, device="cuda") * (0.3 / n ** .5), 1)
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    zero = torch.zeros(1, 1, device="cuda").expand(m, n)
    y, _, _, batch_shape = G._prepare_output(w, l, u, False)
    y_pre = torch.empty_like(y)
    G._sweep_fused(y, l, u, batch_shape, dict(kind=_abi.Q_AFFINE, qmin=-8, qmax=7), (scale, zero), y_pre=y_pre)
    codes = torch.round(y / scale)
    assert codes.min() >= -8 and codes.max() <= 7
    assert torch.equal(y, (torch.clamp(torch.round(y_pre / scale), -8, 7)) * scale)
    e = (y - y_pre).double()
    eye_m, eye_n = torch.eye(m, device="cuda", dtype=torch.float64), torch.eye(n, device="cuda", dtype=torch.float64)
    residual = (y - w).double() - (l.double() + eye_m) @ e @ (u.double() + eye_n)
    assert residual.abs().max().item() < 1e-5 * scale.max().item() * 16
    # same result from a replay of the same call (determinism) and with another far-update width
    y2 = w.clone()
    G._sweep_fused(y2, l, u, batch_shape, dict(kind=_abi.Q_AFFINE, qmin=-8, qmax=7), (scale, zero))
    assert torch.equal(y2, y)


def test_empty_inputs(api):
    """test_gptq_2d.py:149-163: empty batches and matrices return at once and never call the quantizer."""
    G, _ = api
    calls = []
    quantizer = lambda *args, **kwargs: calls.append(args)
    x = torch.randn(6, 10, dtype=torch.float64, device="cuda")
    l, u = torch.randn(6, 6, dtype=torch.float64, device="cuda"), torch.randn(10, 10, dtype=torch.float64, device="cuda")
    for empty, le, ue in ((x.new_empty(0, 6, 10), l, u), (x.new_empty(0, 10), l[:0, :0], u), (x.new_empty(6, 0), l, u[:0, :0])):
        for run in (G.gptq_2d, G.gptq_2d_torch, functools.partial(G.gptq_2d_super_entry, super_entry_shape=(3, 5))):
            assert run(empty, le, ue, quantizer=quantizer).shape == empty.shape
        assert G.gptq_2d(empty, le, ue).shape == empty.shape
        for options in ({}, dict(super_entry_shape=(3, 5))):
            replay = G.capture_gptq_2d(empty, le, ue, quantizer=quantizer, **options)
            assert replay(empty, le, ue).shape == empty.shape
    assert calls == []


def test_large_batch(api, oracle):
    """test_gptq_2d.py:165-172: more batches than a grid's y/z axes hold."""
    G, _ = api
    rng = np.random.default_rng(9)
    x0 = 4 * rng.standard_normal((4, 6))
    l, u = np.tril(.05 * rng.standard_normal((4, 4)), -1), np.triu(.05 * rng.standard_normal((6, 6)), 1)
    offsets = np.arange(70_000)[:, None, None] / 7
    x = cuda(x0) + cuda(offsets)
    z = G.gptq_2d(x, cuda(l), cuda(u))
    z2 = G.gptq_2d_super_entry(x, cuda(l), cuda(u), quantizer=python_round, super_entry_shape=(2, 2), inner_block_size=1)
    for b in (0, 1, 12345, 65535, 65536, 69_999):
        assert torch.equal(z[b].cpu(), torch.from_numpy(oracle.sweep(x0 + offsets[b], l, u)))
        assert torch.equal(z2[b].cpu(), torch.from_numpy(oracle.sweep(x0 + offsets[b], l, u, super_entry_shape=(2, 2))))


def test_cuda_graph(api):
    """test_gptq_2d.py:174-194: replays on new inputs match direct runs, out of place and in place, both engines."""
    G, Q = api
    gen = torch.Generator(device="cuda").manual_seed(4321)
    m, n = 12, 20
    x = 4 * torch.randn(2, m, n, generator=gen, dtype=torch.float64, device="cuda")
    l = torch.tril(.05 * torch.randn(m, m, generator=gen, dtype=torch.float64, device="cuda"), -1)
    u = torch.triu(.05 * torch.randn(n, n, generator=gen, dtype=torch.float64, device="cuda"), 1)
    scale = x.abs() * .05 + .2
    zero = torch.zeros_like(scale)

    def round_to_scale(y_flat, selection, scale, zero, *, out):
        s = scale.flatten(start_dim=-2)
        select = selection if callable(selection) else (lambda t: t[..., selection])
        torch.div(select(y_flat), select(s), out=out).round_().mul_(select(s))

    for quantizer in (Q.affine_quantizer_triton, round_to_scale):
        for shape in (None, (3, 4)):
            if shape is not None and quantizer is not round_to_scale:
                continue
            options = dict(quantizer=quantizer, inner_block_size=2, outer_block_size=4)
            if shape is not None:
                options["super_entry_shape"] = shape
            run = functools.partial(G.gptq_2d if shape is None else G.gptq_2d_super_entry, **options)
            replay = G.capture_gptq_2d(x, l, u, quantizer_inputs=(scale, zero), **options)
            first = replay(x, l, u, scale, zero)
            assert torch.equal(first, run(x, l, u, quantizer_inputs=(scale, zero)))
            second = replay(x + .375, 1.5 * l, .5 * u, 1.5 * scale, zero)
            assert torch.equal(second, run(x + .375, 1.5 * l, .5 * u, quantizer_inputs=(1.5 * scale, zero)))
            assert torch.equal(first, run(x, l, u, quantizer_inputs=(scale, zero)))  # replays return copies
            replay = G.capture_gptq_2d(x, l, u, quantizer_inputs=(scale, zero), inplace=True, **options)
            target = x + .25
            assert replay(target, l, u, scale, zero).data_ptr() == target.data_ptr()
            assert torch.equal(target, run(x + .25, l, u, quantizer_inputs=(scale, zero)))


def test_cuda_graph_pipelined_schedule_fp32(api):
    """The pipelined schedule forks to streams of the library's own and joins back: a capture on the caller's stream
    must hold all of it, and replays must reproduce direct runs bit for bit (the additions have a fixed order)."""
    G, Q = api
    gen = torch.Generator(device="cuda").manual_seed(99)
    m, n = 456, 328
    x = 0.02 * torch.randn(m, n, generator=gen, device="cuda")
    l = torch.tril(torch.randn(m, m, generator=gen, device="cuda") * (0.3 / m ** .5), -1)
    u = torch.triu(torch.randn(n, n, generator=gen, device="cuda") * (0.3 / n ** .5), 1)
    scale = Q.int_abs_max_scale_triton(x, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n).contiguous()
    zero = torch.zeros_like(scale)
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7)
    before = G.SWEEP_SCHEDULE
    try:
        G.SWEEP_SCHEDULE = 3
        direct = G.gptq_2d(x, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
        assert torch.equal(direct, G.gptq_2d(x, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero)))
        replay = G.capture_gptq_2d(x, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
        assert torch.equal(replay(x, l, u, scale, zero), direct)
        shifted = G.gptq_2d(x + 0.01, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
        assert torch.equal(replay(x + 0.01, l, u, scale, zero), shifted)
        assert torch.equal(replay(x, l, u, scale, zero), direct)
    finally:
        G.SWEEP_SCHEDULE = before


def test_quantizer_sees_quantized_values(api):
    """test_gptq_2d.py:113-127: live Y holds the quantized values of all earlier antidiagonals."""
    G, _ = api
    gen = torch.Generator(device="cuda").manual_seed(7)
    x = 4 * torch.randn(12, 8, generator=gen, dtype=torch.float64, device="cuda")
    l = torch.tril(.05 * torch.randn(12, 12, generator=gen, dtype=torch.float64, device="cuda"), -1)
    u = torch.triu(.05 * torch.randn(8, 8, generator=gen, dtype=torch.float64, device="cuda"), 1)
    for run in (functools.partial(G.gptq_2d, inner_block_size=3, outer_block_size=7),
                functools.partial(G.gptq_2d_super_entry, super_entry_shape=(2, 2), inner_block_size=2, outer_block_size=5)):
        earlier = []

        def quantizer(y_flat, selection, *, out):
            select = selection if callable(selection) else lambda t: t[..., selection]
            for earlier_select, earlier_z in earlier:
                assert torch.equal(earlier_select(y_flat), earlier_z)
            torch.round(select(y_flat), out=out)
            earlier.append((select, out.clone()))

        run(x, l, u, quantizer=quantizer)
        assert len(earlier) > 0


def test_unused_triangles_are_never_read_fp32(api):
    """gptq_2d.py:1393-1395: only the entries of L below and of U above the diagonal are read; NaN elsewhere must not
    reach the result on any schedule (the tensor-core operands are sanitised copies)."""
    G, Q = api
    gen = torch.Generator(device="cuda").manual_seed(11)
    m, n = 520, 392
    w = 0.02 * torch.randn(m, n, generator=gen, device="cuda")
    l = torch.tril(torch.randn(m, m, generator=gen, device="cuda") * (0.3 / m ** .5), -1)
    u = torch.triu(torch.randn(n, n, generator=gen, device="cuda") * (0.3 / n ** .5), 1)
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    zero = torch.zeros(1, 1, device="cuda").expand(m, n)
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7)
    poisoned_l = torch.where(torch.ones_like(l).tril(-1) > 0, l, torch.nan)
    poisoned_u = torch.where(torch.ones_like(u).triu(1) > 0, u, torch.nan)
    before = G.SWEEP_SCHEDULE
    try:
        for schedule in (0, 1, 2, 3):
            G.SWEEP_SCHEDULE = schedule
            clean = G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
            dirty = G.gptq_2d(w, poisoned_l, poisoned_u, quantizer=quantizer, quantizer_inputs=(scale, zero))
            assert torch.isfinite(dirty).all() and torch.equal(clean, dirty)
    finally:
        G.SWEEP_SCHEDULE = before
