"""Full-size runs of the benchmark configurations that are not the headline: one JSON line each.

    python configs.py --config c1        # 4096 x 4096 INT4, 0.1 % outliers at 10 sigma, Hessian factors from 8192 samples
    python configs.py --config c2        # 8192 x 28672, INT3 affine, scale and zero point per group of 128 columns
    python configs.py --config c3        # 4096 x 14336 as [16, 256, 14336], three factors, 2-bit HYB trellis
    python configs.py --config c3 --divide 4   # every dimension but the super-entry shrunk (short run)
    python configs.py --config pack      # INT4 codes of an 8192 x 28672 matrix packed and unpacked
    python configs.py --config prep      # the factor preparation of an 8192 x 8192 layer alone
    python configs.py --config gram      # Hessian-factor accumulation, 8192 samples of 8192 channels
    python configs.py --config viterbi   # the trellis quantizer alone

Seeded synthetic inputs with the shapes and value distributions of the configurations (``synthetic.py``); everything
goes through the public entry points.  Configuration 3 rounds ``(1, 16, 16)`` super-entries of the three-factor problem,
which is the two-sided sweep over ``16 x 16`` super-entries of the ``[n1 n2, n3]`` view with the row factor
``kron(L1, ldl_of_inverse(G2, size=16))`` and the column factor ``ldl_of_inverse(G3, size=16).T``.
"""
from __future__ import annotations

import argparse
import functools
import json
import os
import sys


def _timed(fn):
    import torch

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    out = fn()
    end.record()
    torch.cuda.synchronize()
    return out, begin.elapsed_time(end)


def config1(divide: int, device) -> dict:
    """4096 x 4096 weights with 0.1 % of the entries at 10 sigma, both Hessian factors from 8192 heavy-tailed activation
    samples (sigma_h = 1, 1 % damping), INT4 symmetric per-row fp16 scales: one layer alone, preparation then sweep."""
    import torch

    import gptq_2d as G
    import kron_factors as K
    import quantizer_int as Q
    import synthetic

    m = n = 4096 // divide
    w, g, h = synthetic.make_layer(m, n, seed=1, device=device, samples=8192 // divide, outliers=1e-3)
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    zero = torch.zeros(1, 1, device=device).expand(m, n)
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7)
    l, u = K.feedback_factors_from_grams(g, h, check=True)
    G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))  # module load, streams
    K.feedback_factors_from_grams(g, h)  # the timed call once untimed: its workspace comes from the allocator's cache afterwards
    torch.cuda.synchronize()
    (l, u), prep_ms = _timed(lambda: K.feedback_factors_from_grams(g, h))
    z, sweep_ms = _timed(lambda: G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero)))
    K.check_pending()
    G.check_status(device)
    codes = torch.round(z / scale)
    rtn = torch.clamp(torch.round(w / scale), -8, 7) * scale
    flops = float(m) * n * (m + n - 2)
    return {
        "config": "c1", "shape": [m, n], "quantizer": "INT4 symmetric, per-row fp16 abs-max scales", "outliers": float((w.abs() > 9 * 0.02).float().mean()),
        "prep_ms": prep_ms, "sweep_ms": sweep_ms, "layer_ms": prep_ms + sweep_ms, "sweep_tflops": flops / sweep_ms / 1e9,
        "prep_tflops": 2 * (m ** 3 + n ** 3) / 3 / prep_ms / 1e9, "stages": m + n - 1, "us_per_stage": 1e3 * sweep_ms / (m + n - 1),
        "codes_in_range": bool((codes.min() >= -8) & (codes.max() <= 7)), "finite": bool(torch.isfinite(z).all()),
        "objective_vs_rtn": synthetic.objective(z, w, g, h) / synthetic.objective(rtn, w, g, h),
    }


def config2(divide: int, device) -> dict:
    import torch

    import gptq_2d as G
    import kron_factors as K
    import quantizer_int as Q
    import synthetic

    m, n, group = 8192 // divide, 28672 // divide, 128
    generator = torch.Generator(device=device).manual_seed(2)
    w = 0.015 * torch.randn(m, n, generator=generator, device=device)
    g = synthetic.hessian_factor(m, 8192 // divide, 1.0, 0.01, generator, device)
    h = synthetic.hessian_factor(n, 8192 // divide, 1.0, 0.01, generator, device)
    # min / max scale and zero point per (row, group of 128 input columns), expanded to the full matrix as the reference's
    # affine quantizer wants them (quantizer_int.py:63-107)
    groups = w.view(m, n // group, group)
    lo, hi = groups.amin(-1), groups.amax(-1)
    scale_g = (hi - lo) / 7
    zero_g = torch.round(-lo / scale_g)
    scale = scale_g.repeat_interleave(group, dim=1).contiguous()
    zero = zero_g.repeat_interleave(group, dim=1).contiguous()
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=0, qmax=7)
    K.feedback_factors_from_grams(g[:256, :256].contiguous(), h[:256, :256].contiguous())  # module load, streams
    G.gptq_2d(w[:256, :256].contiguous(), *K.feedback_factors_from_grams(g[:256, :256].contiguous(), g[:256, :256].contiguous()),
              quantizer=quantizer, quantizer_inputs=(scale[:256, :256].contiguous(), zero[:256, :256].contiguous()))
    K.feedback_factors_from_grams(g, h, check=True)  # once untimed: the 30 GB of workspace come from the allocator's cache afterwards
    (l, u), prep_ms = _timed(lambda: K.feedback_factors_from_grams(g, h, check=True))
    G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))
    z, sweep_ms = _timed(lambda: G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero)))
    codes = torch.round(z / scale + zero)
    rtn = (torch.clamp(torch.round(w / scale + zero), 0, 7) - zero) * scale

    def objective(q):  # tr(R^T G R H), float64 accumulation in row blocks
        total = 0.0
        r = q - w
        for start in range(0, m, 1024):
            left = (g[start:start + 1024].double() @ r.double())
            total += (left * (r[start:start + 1024].double() @ h.double())).sum().item()
        return total

    flops = float(m) * n * (m + n - 2)
    return {
        "config": "c2", "shape": [m, n], "quantizer": "INT3 affine, group 128", "prep_ms": prep_ms, "sweep_ms": sweep_ms,
        "sweep_tflops": flops / sweep_ms / 1e9, "prep_tflops": 2 * (m ** 3 + n ** 3) / 3 / prep_ms / 1e9,
        "stages": m + n - 1, "us_per_stage": 1e3 * sweep_ms / (m + n - 1),
        "codes_in_range": bool((codes.min() >= 0) & (codes.max() <= 7)), "finite": bool(torch.isfinite(z).all()),
        "objective_vs_rtn": objective(z) / objective(rtn),
    }


def config3(divide: int, device) -> dict:
    import torch

    import gptq_2d as G
    import kron_factors as K
    import quantizer_trellis as T
    import synthetic

    n1, n2, n3, p, q = 16 // min(divide, 16), 256 // divide, 14336 // divide, 16, 16
    generator = torch.Generator(device=device).manual_seed(3)
    x = torch.randn(n1 * n2, n3, generator=generator, device=device)  # an orthogonal transform of Gaussian weights stays Gaussian
    g1 = synthetic.hessian_factor(n1, 4 * n1, 0.5, 0.01, generator, device)
    g2 = synthetic.hessian_factor(n2, 4 * n2, 0.5, 0.01, generator, device)
    g3 = synthetic.hessian_factor(n3, max(n3 // 2, 1024), 1.0, 0.01, generator, device)
    table = T.hyb(L=16, seed=0, device=device, dtype=torch.float32)
    scale = (x.pow(2).mean().sqrt() / (0.9 * table.pow(2).mean().sqrt())).reshape(())
    quantizer = functools.partial(T.trellis_quantizer_super_entry_triton, table=table, K=2, tail_biting=True)

    def prepare():
        return K.ldl_of_inverse(g1, check=False), K.ldl_of_inverse(g2, size=p, check=False), K.ldl_of_inverse(g3, size=q, check=False)

    prepare()
    (l1, l2, l3), prep_ms = _timed(prepare)
    K.check_pending()
    small = K.gptq_d_sided(x[:64, :64].reshape(2, 32, 64).contiguous(), [l1[:2, :2].contiguous(), l2[:32, :32].contiguous(), l3[:64, :64].contiguous()],
                           quantizer=quantizer, quantizer_inputs=(scale,), super_entry_shape=(p, q))
    assert torch.isfinite(small).all()
    # mode by mode: three factors of n1^2 + n2^2 + n3^2 values, all slabs on the hyper-anti-diagonal schedule
    z3, sweep_ms = _timed(lambda: K.gptq_d_sided(x.view(n1, n2, n3), [l1, l2, l3], quantizer=quantizer, quantizer_inputs=(scale,), super_entry_shape=(p, q)))
    z = z3.view(n1 * n2, n3)
    # the other route: the two-sided super-entry sweep of the [n1 n2, n3] view under the explicit Kronecker row factor
    l, u = torch.kron(l1.contiguous(), l2.contiguous()).contiguous(), l3.T.contiguous()
    z_dense, dense_ms = _timed(lambda: G.gptq_2d_super_entry(x, l, u, quantizer=quantizer, super_entry_shape=(p, q), quantizer_inputs=(scale,)))
    G.check_status(device)
    rows, cols = n1 * n2, n3
    sequences = (rows // p) * (cols // q)
    # the same quantizer without feedback: every super-entry of X coded on its own
    blocks = x.view(rows // p, p, cols // q, q).permute(0, 2, 1, 3).reshape(sequences, p * q)
    coded = torch.cat([T._trellis_quantize((blocks[k:k + 16384] / scale).contiguous(), table, 2, True)[0] for k in range(0, sequences, 16384)])
    direct = (coded * scale).view(rows // p, cols // q, p, q).permute(0, 2, 1, 3).reshape(rows, cols)
    big_g = torch.kron(g1, g2).double()

    def objective(candidate):  # tr(R^T (G1 x G2) R G3), float64
        r = (candidate - x).double()
        return ((big_g @ r) * (r @ g3.double())).sum().item()

    # every value is a table entry times the scale: distance of z / scale to the nearest table value
    sample = (z[: 4 * p] / scale).reshape(-1)[: 1 << 14]
    nearest = (sample[:, None] - table.reshape(-1)[None, :]).abs().amin(dim=1).max().item()
    return {
        "config": "c3", "shape": [n1, n2, n3], "view": [rows, cols], "quantizer": "HYB trellis, L = 16, K = 2, V = 2, tail-biting, 16 x 16 super-entries",
        "prep_ms": prep_ms, "sweep_ms": sweep_ms, "stages": n1 + n2 // p + cols // q - 2, "sequences": sequences,
        "row_factor_values": n1 * n1 + n2 * n2, "kronecker_route": {"sweep_ms": dense_ms, "stages": rows // p + cols // q - 1, "row_factor_values": rows * rows,
                                                                 "objective_vs_direct_coding": None, "values_equal_mode_by_mode": (z_dense == z).double().mean().item()},
        "sequences_per_s": sequences / (sweep_ms * 1e-3), "viterbi_tflops": sequences * 1.174e8 / sweep_ms / 1e9,
        "finite": bool(torch.isfinite(z).all()), "max_distance_to_table_value": nearest,
        "objective_vs_direct_coding": objective(z) / objective(direct), "objective_kronecker_route_vs_direct_coding": objective(z_dense) / objective(direct),
        "direct_coding_relative_mse": ((direct - x).pow(2).mean() / x.pow(2).mean()).item(),
    }


def pack(divide: int, device) -> dict:
    """Packing and unpacking the INT4 codes of an 8192 x 28672 matrix: streaming kernels, bound by HBM bandwidth."""
    import torch

    import packed_codes as P
    import quantizer_int as Q

    m, n = 8192 // divide, 28672 // divide
    generator = torch.Generator(device=device).manual_seed(4)
    w = 0.02 * torch.randn(m, n, generator=generator, device=device)
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16)
    zero = torch.zeros(1, 1, device=device)
    z = torch.clamp(torch.round(w / scale), -8, 7) * scale
    codes = P.pack_codes(z, scale, zero, qmin=-8, bits=4)
    assert torch.equal(P.unpack_codes(codes, scale, zero, qmin=-8, bits=4, n=n), z)
    def timed(fn, repeats=10):  # back to back: the host side of a call hides behind the previous launch
        fn()

        def loop():
            for _ in range(repeats):
                fn()  # the result is dropped at once, so every call reuses the same block of the caching allocator

        return _timed(loop)[1] / repeats

    pack_ms = timed(lambda: P.pack_codes(z, scale, zero, qmin=-8, bits=4))
    unpack_ms = timed(lambda: P.unpack_codes(codes, scale, zero, qmin=-8, bits=4, n=n))
    moved = 4.0 * m * n + 0.5 * m * n + 4.0 * m  # z, codes, one scale per row (either direction)
    peak = 6650.0
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    source = "fallback"
    if os.path.exists(path):
        with open(path) as f:
            peak, source = json.load(f)["hbm_gbs"], "measured"
    return {
        "config": "pack", "shape": [m, n], "bits": 4, "pack_ms": pack_ms, "unpack_ms": unpack_ms, "algorithmic_bytes": moved,
        "pack_gbs": moved / pack_ms / 1e6, "unpack_gbs": moved / unpack_ms / 1e6, "hbm_peak_gbs": peak, "peak_source": source,
        "pack_frac": moved / pack_ms / 1e6 / peak, "unpack_frac": moved / unpack_ms / 1e6 / peak,
        "l2": "inputs and outputs (0.94 GB + 0.12 GB) are larger than L2; ten launches back to back",
    }


def prep(divide: int, device) -> dict:
    """The factor preparation alone: both factors of an 8192 x 8192 layer in shared launches, and one factor."""
    import torch

    import kron_factors as K
    import synthetic

    n = 8192 // divide
    generator = torch.Generator(device=device).manual_seed(5)
    g = synthetic.hessian_factor(n, n, 1.0, 0.01, generator, device)
    h = synthetic.hessian_factor(n, n, 1.0, 0.01, generator, device)
    K.feedback_factors_from_grams(g, h, check=True)
    _, pair_ms = _timed(lambda: K.feedback_factors_from_grams(g, h))
    K.ldl_of_inverse(g)
    l, single_ms = _timed(lambda: K.ldl_of_inverse(g, check=False))
    residual = (l.T.double() @ g.double() @ l.double())
    off = residual - torch.diag(residual.diagonal())
    return {"config": "prep", "n": n, "pair_ms": pair_ms, "single_ms": single_ms, "pair_tflops": 2 * (2 * n ** 3 / 3) / pair_ms / 1e9,
            "single_tflops": (2 * n ** 3 / 3) / single_ms / 1e9,
            "off_diagonal_of_LtGL_relative": (off.abs().max() / residual.diagonal().abs().max()).item()}


def gram(divide: int, device) -> dict:
    """Hessian-factor accumulation h += x^T x / k for 8192 samples of 8192 channels on the tensor cores."""
    import torch

    import kron_factors as K

    n = k = 8192 // divide
    generator = torch.Generator(device=device).manual_seed(6)
    x = torch.randn(k, n, generator=generator, device=device) * torch.exp(torch.randn(n, generator=generator, device=device))
    h = torch.zeros(n, n, device=device)
    K.accumulate_gram(h, x, 1.0 / k)
    want = x.double().T @ x.double() / k
    error = ((h.double() - want).abs().max() / want.abs().max()).item()
    plain = ((x.T @ x / k).double() - want).abs().max().item() / want.abs().max().item()
    _, ms = _timed(lambda: K.accumulate_gram(h, x, 1.0 / k))
    _, torch_ms = _timed(lambda: h.addmm_(x.T, x, alpha=1.0 / k))
    flops = float(n) * (n + 1) * k  # the lower triangle with the diagonal, two flops per multiply-add
    return {"config": "gram", "n": n, "k": k, "ms": ms, "tflops": flops / ms / 1e9, "torch_addmm_ms": torch_ms,
            "relative_error": error, "relative_error_of_torch_fp32": plain}


def viterbi(divide: int, device) -> dict:
    """The trellis quantizer alone: HYB code, L = 16, K = 2, V = 2, tail-biting, 256-weight sequences."""
    import torch

    import quantizer_trellis as T

    table = T.hyb(L=16, seed=0, device=device, dtype=torch.float32)
    generator = torch.Generator(device=device).manual_seed(7)
    out = {"config": "viterbi", "flops_per_sequence": 1.174e8}
    for rows in (148, 296, 4096 // divide):
        x = torch.randn(rows, 256, generator=generator, device=device)
        T._trellis_quantize(x, table, 2, True)
        _, ms = _timed(lambda: T._trellis_quantize(x, table, 2, True))
        out[f"rows_{rows}"] = {"ms": ms, "sequences_per_s": rows / ms * 1e3, "tflops": rows * 1.174e8 / ms / 1e9}
    return out


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--config", required=True, choices=("c1", "c2", "c3", "pack", "prep", "gram", "viterbi"))
    parser.add_argument("--divide", type=int, default=1, help="shrink the dimensions by this factor")
    args = parser.parse_args()
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "gptq-2d_b200"))
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("configs.py needs a CUDA device (B200); there is no CPU path")
    device = torch.device("cuda", 0)
    print(json.dumps({"c1": config1, "c2": config2, "c3": config3, "pack": pack, "prep": prep, "gram": gram, "viterbi": viterbi}[args.config](args.divide, device)))


if __name__ == "__main__":
    main()
