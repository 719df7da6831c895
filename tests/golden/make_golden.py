"""Generate the golden vectors under tests/golden by importing the reference implementation.

Run once in a container that has the reference checked out (set GPTQ2D_REF to its directory):

    GPTQ2D_REF=/path/to/GPTQ-2D python tests/golden/make_golden.py

The reference is PyTorch code that cannot travel with the tests, so its outputs on seeded inputs
are stored here as small ``.npz`` files.  The inputs are stored next to the outputs: nothing in the
tests depends on a random generator reproducing a stream.
"""
import functools
import hashlib
import os
import sys

import numpy as np
import torch

REF = os.environ.get("GPTQ2D_REF")
if not REF:
    raise SystemExit("set GPTQ2D_REF to a checkout of the reference project (its gptq_2d.py is imported from there)")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

import gptq_2d as R  # noqa: E402
import gptq_2d_reference as RR  # noqa: E402
import quantizer_int as QI  # noqa: E402
import quantizer_trellis as QT  # noqa: E402


def instance(m, n, seed, shape=(1, 1), dtype=torch.float64):
    """X and factors whose unused triangles and diagonal blocks are NaN (the idea of test_gptq_2d.py:32-40)."""
    g = torch.Generator().manual_seed(seed)
    x = 4. * torch.randn(m, n, generator=g, dtype=dtype)
    l, u = (.05 * torch.randn(k, k, generator=g, dtype=dtype) for k in (m, n))
    for factor, size, unused in ((l, shape[0], torch.ge), (u, shape[1], torch.le)):
        block = torch.arange(factor.size(0)) // size
        factor[unused(block[None, :], block[:, None])] = torch.nan
    return x, l, u


def unit_factors(l, u, shape=(1, 1)):
    out = []
    for factor, size in ((l.tril(), shape[0]), (u.triu(), shape[1])):
        block = torch.arange(factor.size(-1)) // size
        eye = torch.eye(factor.size(-1), dtype=factor.dtype)
        out.append(torch.where(block[:, None] == block[None, :], eye, factor))
    return out


def hessian(dim, k, sigma, damp, g, dtype=torch.float32):
    x = torch.randn(k, dim, generator=g, dtype=dtype) * torch.exp(sigma * torch.randn(dim, generator=g, dtype=dtype))
    h = x.T @ x / k
    h.diagonal().add_(damp * h.diagonal().mean())
    return h


def save(name, **arrays):
    arrays = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in arrays.items()}
    np.savez_compressed(os.path.join(HERE, name), **arrays)
    print(name, sum(a.nbytes for a in arrays.values()) // 1024, "KiB raw")


def sweep_fp64():
    """test_gptq_2d.py:70-89 shapes: round quantizer vs alg3_super_entry, and a joint abs-max quantizer."""
    cases = (
        (1, 1, (1, 1)), (1, 7, (1, 1)), (7, 1, (1, 1)), (13, 5, (1, 1)), (9, 13, (1, 1)), (65, 97, (1, 1)),
        (8, 12, (2, 4)), (6, 6, (3, 2)), (4, 64, (1, 32)), (12, 8, (4, 4)), (16, 16, (16, 16)), (24, 8, (1, 8)),
        (32, 64, (16, 16)), (96, 160, (16, 16)), (90, 75, (3, 5)),
    )
    out = {"cases": np.array([(m, n, p, q) for m, n, (p, q) in cases])}
    joint = functools.partial(QI.int_abs_max_quantizer_torch, qmin=-2, qmax=1, dtype=torch.bfloat16)
    for k, (m, n, shape) in enumerate(cases):
        x, l, u = instance(m, n, 100 * m + n, shape)
        out[f"x{k}"], out[f"l{k}"], out[f"u{k}"] = x, l, u
        out[f"z_round{k}"] = RR.alg3_super_entry(x, *unit_factors(l, u, shape), super_entry_shape=shape)
        assert R.gptq_2d_super_entry_torch(x, l, u, super_entry_shape=shape).equal(out[f"z_round{k}"])
        out[f"z_absmax{k}"] = R.gptq_2d_super_entry_torch(x, l, u, quantizer=joint, super_entry_shape=shape)
    save("sweep_fp64.npz", **out)


def sweep_batched():
    """test_gptq_2d.py:129-147: broadcast batches with a per-entry scale (affine, zero point 0, no clamp)."""
    def round_to_scale(y_flat, selection, scale, *, out):
        torch.div(y_flat[..., selection], scale[..., selection], out=out).round_().mul_(scale[..., selection])

    out = {}
    for k, (m, n) in enumerate(((12, 8), (9, 15), (33, 70))):
        x, l, u = instance(m, n, 10 * m + n)
        x = torch.stack((x, x + .25))[:, None, :, :]
        l = torch.stack((l, .5 * l, 2. * l))[None, :, :, :]
        scale = x.abs().flatten(start_dim=-2) * .05 + .2
        lu, uu = unit_factors(l, u)
        z = R.gptq_2d_torch(x, lu, uu, quantizer=round_to_scale, quantizer_inputs=(scale,))
        out[f"x{k}"], out[f"l{k}"], out[f"u{k}"], out[f"scale{k}"], out[f"z{k}"] = x, l, u, scale.unflatten(-1, (m, n)), z
    out["count"] = 3
    save("sweep_batched_fp64.npz", **out)


def quartic_64():
    """The first benchmark configuration's 64 x 64 check: the sweep against the quartic vectorized-GPTQ reference
    (gptq_2d_reference.py:360-382) with the coordinate-dependent clipped codebook of :354-357."""
    m = n = 64
    a, b, x = RR._random_instance((m, n), 1000 * m + 10 * n, "cpu")
    l, u = RR.feedback_factors(a, b)
    z = RR._vectorized_alg1(x, a, b, Q=RR._coordinate_round)
    assert RR.alg3(x, l, u, Q=RR._coordinate_round).equal(z)
    i, j = torch.arange(m)[:, None], torch.arange(n)
    scale = (2. ** ((i + 2 * j) % 3 - 1)).double()
    save("quartic_64_fp64.npz", x=x, l=l, u=u, scale=scale, z=z, qmin=-3., qmax=2.)


def config0_fp32():
    """The first benchmark configuration: 256 x 256 fp32 INT4 with per-row fp16 abs-max scales, seed 0, through gptq_2d_torch."""
    g = torch.Generator().manual_seed(0)
    for n in (64, 256):
        w = 0.02 * torch.randn(n, n, generator=g)
        gm, hm = hessian(n, 1024, .5, .01, g), hessian(n, 1024, .5, .01, g)
        l, u = RR.ldl_of_inverse(gm).contiguous(), RR.ldl_of_inverse(hm).T.contiguous()
        scale = QI.int_abs_max_scale_torch(w, qmin=-8, qmax=7, dtype=torch.float16)
        full = scale.expand(n, n).contiguous()
        quantizer = functools.partial(QI.affine_quantizer_torch, qmin=-8, qmax=7)
        z = R.gptq_2d_torch(w, l, u, quantizer=quantizer, quantizer_inputs=(full, torch.zeros_like(w)))
        z_one_sided = R.gptq_2d_torch(w, torch.eye(n), u, quantizer=quantizer, quantizer_inputs=(full, torch.zeros_like(w)))
        save(f"config0_{n}_fp32.npz", w=w, g=gm, h=hm, l=l, u=u, scale=scale, z=z, z_one_sided=z_one_sided)


def quantizers():
    g = torch.Generator().manual_seed(3)
    out = {}
    for name, dt in (("f32", torch.float32), ("f64", torch.float64)):
        x = 4. * torch.randn(96, 32, generator=g, dtype=dt)
        x[1] = 0.
        x[2] *= 1e-38
        x[3] *= 1e-6
        x[4] *= 3e4
        out[f"x_{name}"] = x
        for hname, hd in (("fp16", torch.float16), ("bf16", torch.bfloat16)):
            out[f"scale_{name}_{hname}"] = QI.int_abs_max_scale_torch(x, qmin=-8, qmax=7, dtype=hd)
            for qmin, qmax in ((-2, 1), (-8, 7), (-128, 127)):
                o = torch.empty(96, 1, 32, dtype=dt)
                QI.int_abs_max_quantizer_torch(x, lambda t: t.unflatten(-1, (1, 32)), out=o, qmin=qmin, qmax=qmax, dtype=hd)
                out[f"absmax_{name}_{hname}_{qmax}"] = o
        y = 4. * torch.randn(2, 3, 35, generator=g, dtype=dt)
        scale = .1 + torch.rand(1, 5, 7, generator=g, dtype=dt)
        zero = torch.randint(-2, 3, (2, 1, 5, 7), generator=g).to(dt)
        o = torch.empty(2, 3, 35, dtype=dt)
        QI.affine_quantizer_torch(y, slice(0, 35, 1), scale, zero, qmin=-3, qmax=4, out=o)
        out[f"aff_y_{name}"], out[f"aff_scale_{name}"], out[f"aff_zero_{name}"], out[f"aff_out_{name}"] = y, scale, zero, o
    save("quantizers.npz", **out)


def sha(t):
    return np.frombuffer(hashlib.sha256(t.contiguous().numpy().tobytes()).digest(), dtype=np.uint8)


def trellis():
    g = torch.Generator().manual_seed(4)
    out = {}
    shapes = ((5, 1, 1, 7), (4, 1, 2, 8), (6, 1, 2, 14), (10, 2, 2, 64), (9, 3, 1, 21), (12, 4, 2, 40), (7, 1, 1, 1))
    k = 0
    for (L, K, V, T) in shapes:
        for name, dt in (("f32", torch.float32), ("f64", torch.float64)):
            table = torch.randn(1 << L, V, generator=g, dtype=dt)
            x = torch.randn(37, T, generator=g, dtype=dt)
            out[f"x{k}"], out[f"table{k}"], out[f"K{k}"] = x, table, K
            for tb in (0, 1):
                values, states = QT._trellis_quantize_torch(x, table, K, bool(tb))
                out[f"values{k}_{tb}"], out[f"states{k}_{tb}"] = values, states
            k += 1
    table = torch.randint(-3, 4, (1 << 8, 2), generator=g).float()  # many ties
    x = torch.randint(-3, 4, (40, 64), generator=g).float()
    out[f"x{k}"], out[f"table{k}"], out[f"K{k}"] = x, table, 2
    for tb in (0, 1):
        out[f"values{k}_{tb}"], out[f"states{k}_{tb}"] = QT._trellis_quantize_torch(x, table, 2, bool(tb))
    k += 1
    out["count"] = k
    # the shipped codes at L = 16 with 256-value sequences (quantizer_trellis.py:476-479)
    tlut = QT._gaussian_codebook(1 << 9)
    out["tlut"] = tlut
    codes = {"hyb": QT.hyb(), "one_mad": QT.one_mad(), "three_inst": QT.three_inst()}
    for name, table in codes.items():
        out[f"sha_{name}"] = sha(table)
        out[f"head_{name}"] = table[:64]
    for name, Ks in (("hyb", (2, 3, 4)), ("one_mad", (2, 4)), ("three_inst", (2,))):
        x = torch.randn(6, 256, generator=g)
        out[f"code_x_{name}"] = x
        for K in Ks:
            values, states = QT._trellis_quantize_torch(x, codes[name], K, True)
            out[f"code_values_{name}_{K}"], out[f"code_states_{name}_{K}"] = values, states
    save("trellis.npz", **out)


def trellis_sweep():
    """test_gptq_2d.py:91-111: a trellis rounds each 16 x 16 super-entry jointly inside the sweep."""
    table = torch.randn(1 << 8, 2, generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    x, l, u = instance(32, 64, 7, (16, 16))
    scale = torch.tensor(4., dtype=torch.float64)
    quantizer = functools.partial(QT.trellis_quantizer_super_entry_torch, table=table, K=2)
    z = R.gptq_2d_super_entry_torch(x, l, u, quantizer=quantizer, super_entry_shape=(16, 16), quantizer_inputs=(scale,))
    save("trellis_sweep_fp64.npz", x=x, l=l, u=u, table=table, scale=scale, z=z, K=2)


def factors():
    g = torch.Generator().manual_seed(11)
    out = {}
    for n in (1, 7, 64, 200):
        gm = hessian(n, 4 * n + 8, 1., .01, g, torch.float64)
        out[f"g{n}"], out[f"l{n}"] = gm, RR.ldl_of_inverse(gm)
    gm = hessian(48, 256, 1., .01, g, torch.float64)
    out["g48"] = gm
    for size in (1, 2, 4, 16):
        out[f"l48_{size}"] = RR.ldl_of_inverse(gm, size)
    gm = hessian(256, 1024, 1., .01, g, torch.float32)
    out["g256_f32"], out["l256_f32"] = gm, RR.ldl_of_inverse(gm)
    save("factors.npz", **out)


def d_sided():
    """gptq_2d_reference.py:450-478: N-factor rounding against Algorithm 1 on the explicit Kronecker Gram."""
    out = {}
    shapes = ((7,), (4, 6), (1, 4, 3), (3, 4, 5), (2, 3, 2, 3), (4, 8, 16))
    for k, shape in enumerate(shapes):
        *bases, x = RR._random_instance(shape, k, "cpu")
        factors_ = [RR.ldl_of_inverse(a.t() @ a) for a in bases]
        out[f"x{k}"] = x
        for d, f in enumerate(factors_):
            out[f"l{k}_{d}"] = f
        out[f"z{k}"] = RR.alg4(x, factors_)
    out["count"] = len(shapes)
    save("d_sided_fp64.npz", **out)


def factors_fp32_large():
    """float32 ``ldl_of_inverse`` of heavy-tailed Grams at n = 1024 and 2048 (the reference's LAPACK path), next to its
    own float64 result on the same float32-valued matrix.  The Grams come from a recipe whose float32 values are the
    same bits everywhere (``oracle.dyadic_gram``), so only a sample of rows of each factor is stored."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import oracle

    out = {}
    for n in (1024, 2048):
        gram = oracle.dyadic_gram(n, seed=n)
        rows = np.unique(np.concatenate([np.arange(0, n, n // 32), np.arange(n - 8, n)]))
        l32 = RR.ldl_of_inverse(torch.from_numpy(gram)).numpy()
        l64 = RR.ldl_of_inverse(torch.from_numpy(gram).double()).numpy()
        out[f"rows{n}"], out[f"l32_{n}"], out[f"l64_{n}"] = rows, l32[rows], l64[rows]
        out[f"gram_sum{n}"] = gram.astype(np.float64).sum()
        out[f"gap{n}"] = np.abs(l32.astype(np.float64) - l64).max()
        out[f"lmax{n}"] = np.abs(l64).max()
    save("factors_fp32_large.npz", **out)


def config1_small():
    """The second benchmark configuration's distributions (0.1 % outliers at 10 sigma, sigma_h = 1 Hessian factors) at
    256 x 384 through the reference's gptq_2d_torch in float64: the INT4 codes, on float32-valued inputs."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import oracle

    m, n = 256, 384
    w, g, h = oracle.config1_layer(m, n, seed=41)
    l = RR.ldl_of_inverse(torch.from_numpy(g).double()).float().double().contiguous()
    u = RR.ldl_of_inverse(torch.from_numpy(h).double()).float().double().T.contiguous()
    scale = QI.int_abs_max_scale_torch(torch.from_numpy(w), qmin=-8, qmax=7, dtype=torch.float16)
    full = scale.double().expand(m, n).contiguous()
    zero = torch.zeros(m, n, dtype=torch.float64)
    quantizer = functools.partial(QI.affine_quantizer_torch, qmin=-8, qmax=7)
    z = R.gptq_2d_torch(torch.from_numpy(w).double(), l, u, quantizer=quantizer, quantizer_inputs=(full, zero))
    save("config1_small_fp64.npz", scale=scale, codes=torch.round(z / full).to(torch.int8), l=l.float(), u=u.float(),
         w_sum=np.float64(w.astype(np.float64).sum()))


if __name__ == "__main__":
    torch.set_num_threads(8)
    steps = dict(sweep_fp64=sweep_fp64, sweep_batched=sweep_batched, quartic_64=quartic_64, config0_fp32=config0_fp32,
                 quantizers=quantizers, trellis=trellis, trellis_sweep=trellis_sweep, factors=factors, d_sided=d_sided,
                 factors_fp32_large=factors_fp32_large, config1_small=config1_small)
    for name in sys.argv[1:] or steps:  # name the steps to (re)generate; all of them by default
        steps[name]()
