"""Reduced-size versions of the benchmark configurations 2 and 3 against the oracle (the full sizes are measured by the
benchmark and the layer-set driver; parity is checked here where the oracle finishes in seconds)."""
import functools

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_config2_int3_affine_groups(oracle):
    """Config 2 shape family: rectangular (down-projection aspect), INT3 affine with min/max scale and zero point per
    group of 128 input columns; teacher-forced fp32 replay against the oracle's fp64 decisions."""
    import gptq_2d as G
    import kron_factors as K
    import quantizer_int as Q

    rng = np.random.default_rng(2)
    m, n, group = 512, 1792, 128
    w = (0.015 * rng.standard_normal((m, n))).astype(np.float32)
    lo, hi = w.reshape(m, n // group, group).min(-1), w.reshape(m, n // group, group).max(-1)
    scale_g = ((hi - lo) / 7).astype(np.float32)
    zero_g = np.rint(-lo / scale_g).astype(np.float32)
    scale, zero = np.repeat(scale_g, group, axis=1), np.repeat(zero_g, group, axis=1)
    gen = torch.Generator(device="cuda").manual_seed(3)

    def factor(dim):
        x = torch.randn(2 * dim, dim, generator=gen, device="cuda", dtype=torch.float64) * torch.exp(torch.randn(dim, generator=gen, device="cuda", dtype=torch.float64))
        h = x.T @ x / (2 * dim)
        h.diagonal().add_(0.01 * h.diagonal().mean())
        return K.ldl_of_inverse(h)

    l64, u64 = factor(m), factor(n).T.contiguous()
    l, u = l64.float().cpu().numpy(), u64.float().cpu().numpy()
    z_star = oracle.sweep(w.astype(np.float64), l.astype(np.float64), u.astype(np.float64), kind=oracle.Q_AFFINE,
                          scale=scale.astype(np.float64), zero_point=zero.astype(np.float64), qmin=0, qmax=7)
    # free run: codes in range, objective close to the oracle's
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=0, qmax=7)
    z = G.gptq_2d(cuda(w), cuda(l), cuda(u), quantizer=quantizer, quantizer_inputs=(cuda(scale), cuda(zero)))
    codes = torch.round(z / cuda(scale) + cuda(zero))
    assert codes.min() >= 0 and codes.max() <= 7
    # teacher-forced: the engine's pre-rounding values give the oracle's codes except next to ties
    _, y_pre = G.gptq_2d_forced(cuda(w), cuda(l), cuda(u), cuda(z_star.astype(np.float32)))
    t = y_pre.cpu().numpy().astype(np.float64) / scale + zero
    would_be = np.clip(np.rint(t), 0, 7)
    star = np.rint(z_star / scale + zero)
    mismatch = would_be != star
    assert mismatch.mean() <= 1e-3
    assert (np.abs(np.abs(t - np.floor(t)) - 0.5)[mismatch] <= 1e-5).all()
    agree = (codes.cpu().numpy() == star).mean()
    assert agree > 0.5  # free-running fp32 trajectories drift apart; the bound only guards against gross errors


def test_config3_trellis_three_factors(oracle):
    """Config 3 shape family: a [n1, n2, n3] tensor with one factor per mode, rounded by a 2-bit trellis over
    (1, 16, 16) super-entries = 16 x 16 super-entries of the [n1 n2, n3] view with the row factor
    kron(L1, block-normalised L2); values must equal the oracle's (fp64, bit for bit)."""
    import gptq_2d as G
    import kron_factors as K
    import quantizer_trellis as T

    rng = np.random.default_rng(3)
    n1, n2, n3 = 3, 32, 48
    x = rng.standard_normal((n1, n2, n3))
    def gram(dim):
        a = rng.standard_normal((2 * dim, dim))
        return a.T @ a / (2 * dim) + 0.05 * np.eye(dim)
    l1 = K.ldl_of_inverse(cuda(gram(n1)))
    l2 = K.ldl_of_inverse(cuda(gram(n2)), size=16)
    l3 = K.ldl_of_inverse(cuda(gram(n3)), size=16)
    row_factor = torch.kron(l1.contiguous(), l2.contiguous())
    table = cuda(rng.standard_normal((1 << 8, 2)))
    scale = torch.tensor(1.1, dtype=torch.float64, device="cuda")
    quantizer = functools.partial(T.trellis_quantizer_super_entry_triton, table=table, K=2)
    z = G.gptq_2d_super_entry(cuda(x.reshape(n1 * n2, n3)), row_factor, l3.T.contiguous(), quantizer=quantizer,
                              super_entry_shape=(16, 16), quantizer_inputs=(scale,))
    expected = oracle.sweep(x.reshape(n1 * n2, n3), row_factor.cpu().numpy(), l3.T.cpu().numpy(), kind=oracle.Q_TRELLIS,
                            super_entry_shape=(16, 16), scale=1.1, table=table.cpu().numpy(), K=2)
    assert torch.equal(z.cpu(), torch.from_numpy(expected))
    # the same problem mode by mode: three factors of 3^2, 32^2 and 48^2 values, no Kronecker product
    z3 = K.gptq_d_sided(cuda(x), [l1, l2, l3], quantizer=quantizer, quantizer_inputs=(scale,), super_entry_shape=(16, 16))
    assert torch.equal(z3.cpu(), torch.from_numpy(expected).reshape(n1, n2, n3))


def test_layer_pipeline_equals_plain_calls():
    """Two layers in flight (preparation of one beside the sweep of the other, host buffers in and out) give exactly
    what one call after the other gives."""
    import gptq_2d as G
    import kron_factors as K
    import layer_set
    import quantizer_int as Q
    import synthetic

    device = torch.device("cuda", 0)
    layers = [synthetic.make_layer(392, 520, seed=11 + k, device=device, samples=1024, sigma_h=0.5) for k in range(3)]
    expected = []
    for w, g, h in layers:
        l, u = K.feedback_factors_from_grams(g, h)
        scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand_as(w)
        zero = torch.zeros(1, 1, device=device).expand_as(w)
        expected.append(G.gptq_2d(w, l, u, quantizer=functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7), quantizer_inputs=(scale, zero)))
    pipeline = layer_set.LayerPipeline(device)
    got = [pipeline.quantize(w, g, h) for w, g, h in layers]
    torch.cuda.synchronize()
    for a, b in zip(got, expected):
        assert torch.equal(a, b)
    host = [[t.cpu().pin_memory() for t in layer] for layer in layers]
    outs = [torch.empty_like(h[0]).pin_memory() for h in host]
    done = [pipeline.quantize_from_host(hw, hg, hh, out) for (hw, hg, hh), out in zip(host, outs)]
    for event, out, want in zip(done, outs, expected):
        event.synchronize()
        assert torch.equal(out, want.cpu())
    # the compact transfer format: packed lower triangles of the symmetric Hessian factors in, packed INT4 codes and
    # fp16 row scales out; decoding the codes gives the same matrices
    import packed_codes as P

    packed = [[hw, P.pack_symmetric(hg).pin_memory(), P.pack_symmetric(hh).pin_memory()] for hw, hg, hh in host]
    assert packed[0][1].numel() == 392 * 393 // 2
    codes = [torch.empty(392, 260, dtype=torch.uint8).pin_memory() for _ in host]
    scales = [torch.empty(392, dtype=torch.float16).pin_memory() for _ in host]
    done = [pipeline.quantize_from_host_packed(hw, hg, hh, c, s) for (hw, hg, hh), c, s in zip(packed, codes, scales)]
    for event, c, s, want in zip(done, codes, scales, expected):
        event.synchronize()
        back = P.unpack_codes(c.cuda(), s.cuda().float()[:, None], torch.zeros((), device=device), qmin=-8, bits=4, n=520)
        assert torch.equal(back, want)
    pipeline.check()
    full = torch.randn(77, 77, device=device, dtype=torch.float64)
    full = full + full.T
    assert torch.equal(P.unpack_symmetric(P.pack_symmetric(full), 77), full)


def test_shared_input_factors_equal_separate_calls():
    """A group of matrices that shares its input-side factor (q, k, v of a block) gets U once; every member's result is
    what the plain per-matrix calls give with the same Hessian factors."""
    import functools

    import gptq_2d as G
    import kron_factors as K
    import layer_set
    import quantizer_int as Q
    import synthetic

    device = torch.device("cuda", 0)
    items = [i for i in layer_set.layer_list(1, divide=16, shared_inputs=True) if i["name"] in ("q", "k", "v")]
    assert len({i["group"] for i in items}) == 1
    pipeline = layer_set.LayerPipeline(device)
    fetch = [layer_set.quantize_matrix(item, device, pipeline) for item in items]
    stats = [f() for f in fetch]
    pipeline.check()
    assert all(s["finite"] and s["codes_in_range"] and s["factors_ok"] for s in stats)
    for item, got in zip(items, stats):
        m, n = item["m"], item["n"]
        w, g, h = synthetic.make_layer(m, n, seed=item["seed"], device=device, samples=min(8192, max(m, n)), input_seed=item["input_seed"])
        l, u = K.feedback_factors_from_grams(g, h, check=True)
        scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
        zero = torch.zeros(1, 1, device=device).expand(m, n)
        z = G.gptq_2d(w, l, u, quantizer=functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7), quantizer_inputs=(scale, zero))
        assert got["code_sum"] == torch.round(z / scale).double().sum().item()
