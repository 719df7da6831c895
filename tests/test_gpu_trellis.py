"""GPU parity of the trellis quantizer: values and states must equal the reference's bit for bit."""
import functools
import hashlib

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    import quantizer_trellis
    return quantizer_trellis


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_golden_searches(T):
    """quantizer_trellis.py:465-475 shapes, fp32 and fp64, with and without tail-biting, many-ties table included."""
    g = load_golden("trellis.npz")
    for k in range(int(g["count"])):
        x, table, K = cuda(g[f"x{k}"]), cuda(g[f"table{k}"]), int(g[f"K{k}"])
        for tb in (0, 1):
            values, states = T._trellis_quantize(x, table, K, bool(tb))
            assert torch.equal(values.cpu(), torch.from_numpy(g[f"values{k}_{tb}"])), (k, tb)
            assert torch.equal(states.cpu(), torch.from_numpy(g[f"states{k}_{tb}"])), (k, tb)
            shift, V = K * table.size(1), table.size(1)
            shared = (table.size(0) >> shift) - 1
            assert ((states[..., 1:] >> shift) == (states[..., :-1] & shared)).all()
            assert not tb or ((states[..., 0] >> shift) == (states[..., -1] & shared)).all()
            assert torch.equal(values, table[states, :].flatten(start_dim=-2))


def test_codes_and_long_sequences(T):
    """The shipped codes at L = 16 with 256-value sequences (quantizer_trellis.py:476-479); tables equal the reference's."""
    g = load_golden("trellis.npz")
    tables = {"hyb": T.hyb(device="cuda"), "one_mad": T.one_mad(device="cuda"), "three_inst": T.three_inst(device="cuda")}
    assert torch.equal(T._gaussian_codebook(1 << 9, device="cuda").cpu(), torch.from_numpy(g["tlut"]))
    for name, table in tables.items():
        digest = np.frombuffer(hashlib.sha256(table.cpu().contiguous().numpy().tobytes()).digest(), dtype=np.uint8)
        assert np.array_equal(digest, g[f"sha_{name}"]), name
        assert T.__dict__[name](device="cuda", dtype=torch.float64).equal(table.double())
    for name, Ks in (("hyb", (2, 3, 4)), ("one_mad", (2, 4)), ("three_inst", (2,))):
        x = cuda(g[f"code_x_{name}"])
        for K in Ks:
            values, states = T._trellis_quantize(x, tables[name], K, True)
            assert torch.equal(values.cpu(), torch.from_numpy(g[f"code_values_{name}_{K}"])), (name, K)
            assert torch.equal(states.cpu(), torch.from_numpy(g[f"code_states_{name}_{K}"])), (name, K)


@pytest.mark.parametrize("rows", [1, 37, 300, 700])
def test_many_rows_against_oracle(T, oracle, rows):
    """Row counts that select 1, 2 and 4 sequences per CTA, ragged against the CTA's share."""
    rng = np.random.default_rng(rows)
    table = rng.standard_normal((1 << 10, 2)).astype(np.float32)
    x = rng.standard_normal((rows, 64)).astype(np.float32)
    scale = (0.5 + rng.random(rows)).astype(np.float32)
    expected_values, expected_states = oracle.trellis_quantize(x, table, 2, True)
    out = torch.empty(rows, 64, device="cuda")
    states = torch.empty(rows, 32, dtype=torch.int64, device="cuda")
    T._trellis_quantize_triton(cuda(x), cuda(table), 2, True, out=out, scale=cuda(scale), states=states)
    assert torch.equal(states.cpu(), torch.from_numpy(expected_states))
    assert torch.equal(out.cpu(), torch.from_numpy(expected_values * scale[:, None]))
    if rows < 6:
        return
    shaped = torch.empty(2, 3, 64, device="cuda")
    T._trellis_quantize_triton(cuda(x[:6].reshape(2, 3, 64)), cuda(table), 2, False, out=shaped, scale=torch.ones(2, 3, device="cuda"))
    assert torch.equal(shaped.cpu().reshape(6, 64), torch.from_numpy(oracle.trellis_quantize(x[:6], table, 2, False)[0]))


def test_super_entry_quantizer_scales_and_graph(T, oracle):
    """quantizer_trellis.py:482-519: a scale per matrix or per batch; replays of a captured quantizer on new inputs."""
    table = T.hyb(device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(5)
    y_flat = torch.randn(2, 6 * 16 * 16, generator=gen, device="cuda")
    select = lambda t: t.unflatten(-1, (6, 16, 16))
    for scale in (torch.tensor(1.3, device="cuda"), torch.tensor([1.3, .7], device="cuda")[:, None, None, None]):
        out = torch.empty(2, 6, 16, 16, device="cuda")
        T.trellis_quantizer_super_entry_triton(y_flat, select, scale, out=out, table=table, K=2)
        x = (select(y_flat) / scale).flatten(start_dim=-2)
        values, _ = oracle.trellis_quantize(x.cpu().numpy(), table.cpu().numpy(), 2, True)
        expected = torch.from_numpy(values).view(2, 6, 16, 16) * scale.cpu()
        assert torch.equal(out.cpu(), expected)
    y_one, scale = torch.randn(6 * 16 * 16, generator=gen, device="cuda"), torch.tensor(1.3, device="cuda")
    out = torch.empty(6, 16, 16, device="cuda")
    run = lambda: T.trellis_quantizer_super_entry_triton(y_one, select, scale, out=out, table=table, K=2)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        run()
    for factor in (1., 2.5):
        new_y, new_scale = factor * torch.randn(6 * 16 * 16, generator=gen, device="cuda"), torch.tensor(.9 * factor, device="cuda")
        y_one.copy_(new_y)
        scale.copy_(new_scale)
        graph.replay()
        expected = torch.empty_like(out)
        T.trellis_quantizer_super_entry_triton(new_y, select, new_scale, out=expected, table=table, K=2)
        assert torch.equal(out, expected)


def test_trellis_inside_the_sweep(T):
    """test_gptq_2d.py:91-111: each 16 x 16 super-entry rounded as one sequence inside the sweep, also replayed from a graph."""
    import gptq_2d as G

    g = load_golden("trellis_sweep_fp64.npz")
    x, l, u, table, scale = (cuda(g[k]) for k in ("x", "l", "u", "table", "scale"))
    options = dict(quantizer=functools.partial(T.trellis_quantizer_super_entry_triton, table=table, K=int(g["K"])), super_entry_shape=(16, 16))
    expected = torch.from_numpy(g["z"])
    for blocks in (dict(), dict(inner_block_size=2, outer_block_size=5), dict(inner_block_size=0)):
        z = G.gptq_2d_super_entry(x, l, u, quantizer_inputs=(scale,), **options, **blocks)
        assert torch.equal(z.cpu(), expected)
    replay = G.capture_gptq_2d(x, l, u, quantizer_inputs=(scale,), **options)
    assert torch.equal(replay(x, l, u, scale).cpu(), expected)
    again = replay(x + .375, 1.5 * l, .5 * u, 2 * scale)
    assert torch.equal(again, G.gptq_2d_super_entry(x + .375, 1.5 * l, .5 * u, quantizer_inputs=(2 * scale,), **options))


def test_stored_paths_match_the_oracle_and_decode_back(T, oracle):
    """The search's packed output: the bytes are the oracle's packing of the golden states, and decoding them gives back
    the values and the states bit for bit (fp32 and fp64, tail-biting strings and strings with a header, scaled)."""
    import packed_codes as P

    g = load_golden("trellis.npz")
    checked = 0
    for k in range(int(g["count"])):
        x, table, K = cuda(g[f"x{k}"]), cuda(g[f"table{k}"]), int(g[f"K{k}"])
        L, V = table.size(0).bit_length() - 1, table.size(1)
        for tb in (0, 1):
            states = g[f"states{k}_{tb}"]
            if tb and states.shape[-1] * K * V < L:
                continue
            scale = torch.linspace(0.5, 2.0, x.shape[:-1].numel(), device="cuda", dtype=x.dtype).reshape(x.shape[:-1])
            values, codes = P.trellis_quantize_packed(x, table, K, bool(tb), scale=scale)
            assert torch.equal(values, cuda(g[f"values{k}_{tb}"]) * scale[..., None])
            assert np.array_equal(codes.cpu().numpy(), oracle.trellis_pack(states, L, K, V, bool(tb))), (k, tb)
            back, back_states = P.trellis_decode(codes, table, K, x.size(-1), bool(tb), scale=scale, dtype=x.dtype, return_states=True)
            assert torch.equal(back, values) and torch.equal(back_states.cpu(), torch.from_numpy(states))
            checked += 1
    assert checked >= 6
    # the benchmark's code: HYB, L = 16, 2 bits per weight, 256-weight tail-biting sequences -> 64 bytes each
    table = T.hyb(device="cuda")
    x = torch.randn(40, 256, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    values, codes = P.trellis_quantize_packed(x, table, 2)
    assert codes.shape == (40, 64)
    want, states = T._trellis_quantize(x, table, 2, True)
    assert torch.equal(values, want)
    assert torch.equal(P.trellis_decode(codes, table, 2, 256), values)
    assert np.array_equal(codes.cpu().numpy(), oracle.trellis_pack(states.cpu().numpy(), 16, 2, 2, True))


def test_sweep_stores_its_trellis_paths(T):
    """A trellis sweep that also returns the stored paths: the result is the plain sweep's, and every super-entry of Z is
    recovered from its 8 bytes (16 x 4 super-entries of 2-bit weights)."""
    import gptq_2d as G
    import packed_codes as P

    g = load_golden("trellis_sweep_fp64.npz")
    x, l, u, table = cuda(g["x"]), cuda(g["l"]), cuda(g["u"]), cuda(g["table"])
    scale = cuda(g["scale"])
    z, codes = P.gptq_2d_trellis_packed(x, l, u, scale, table=table, K=int(g["K"]), super_entry_shape=(16, 16))
    assert torch.equal(z.cpu(), torch.from_numpy(g["z"]))
    m, n = x.shape
    blocks = z.reshape(m // 16, 16, n // 16, 16).permute(0, 2, 1, 3).reshape(m // 16, n // 16, 256)
    assert torch.equal(P.trellis_decode(codes, table, int(g["K"]), 256, scale=scale, dtype=x.dtype), blocks)
    # a batch with one scale per matrix
    xb = torch.stack([x, 0.5 * x])
    scales = torch.tensor([1.1, 0.7], dtype=x.dtype, device="cuda").reshape(2, 1, 1, 1)
    zb, cb = P.gptq_2d_trellis_packed(xb, l, u, scales, table=table, K=int(g["K"]), super_entry_shape=(16, 16))
    quantizer = functools.partial(T.trellis_quantizer_super_entry_triton, table=table, K=int(g["K"]))
    for b in range(2):
        want = G.gptq_2d_super_entry(xb[b], l, u, quantizer=lambda *a, **k: quantizer(*a, **k), super_entry_shape=(16, 16), quantizer_inputs=(scales[b, 0, 0, 0],))
        assert torch.equal(zb[b], want)
    blocks = zb.reshape(2, m // 16, 16, n // 16, 16).permute(0, 1, 3, 2, 4).reshape(2, m // 16, n // 16, 256)
    per_entry = scales.reshape(2, 1, 1).expand(2, m // 16, n // 16)
    assert torch.equal(P.trellis_decode(cb, table, int(g["K"]), 256, scale=per_entry, dtype=x.dtype), blocks)
