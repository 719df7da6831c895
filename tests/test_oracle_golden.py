"""The CPU oracle against the golden vectors generated from the reference (tests/golden/make_golden.py)."""
import hashlib

import numpy as np

from conftest import load_golden


def test_affine_known_answers(oracle):
    # quantizer_int.py:475-488: expected [0, 2, -10] and, clamped to -2..2, [0, 1, -6]
    y, scale, zero = np.array([.5, 1.75, -9.]), np.array([1., .5, 2.]), np.array([0., 0., 1.])
    assert np.array_equal(oracle.affine_quantize(y, scale, zero), [0., 2., -10.])
    assert np.array_equal(oracle.affine_quantize(y, scale, zero, -2, 2), [0., 1., -6.])


def test_absmax_scale_known_answer(oracle):
    # quantizer_int.py:532-533: [[1.], [.4 rounded to fp16]]
    scale = oracle.absmax_scale(np.array([[0., 0.], [3., -1.5]], dtype=np.float32), -8, 7, oracle.FP16)
    assert np.array_equal(scale, np.array([[1.], [np.float32(np.float16(.4))]], dtype=np.float32))


def test_quantizers_golden(oracle):
    g = load_golden("quantizers.npz")
    for name in ("f32", "f64"):
        x = g[f"x_{name}"]
        for hname, half in (("fp16", oracle.FP16), ("bf16", oracle.BF16)):
            assert np.array_equal(oracle.absmax_scale(x, -8, 7, half), g[f"scale_{name}_{hname}"])
            for qmin, qmax in ((-2, 1), (-8, 7), (-128, 127)):
                assert np.array_equal(oracle.absmax_quantize(x, qmin, qmax, half), g[f"absmax_{name}_{hname}_{qmax}"][:, 0, :], equal_nan=True)
        y, scale, zero = g[f"aff_y_{name}"], g[f"aff_scale_{name}"].reshape(1, 1, 35), g[f"aff_zero_{name}"].reshape(2, 1, 35)
        assert np.array_equal(oracle.affine_quantize(y, scale, zero, -3, 4), g[f"aff_out_{name}"])


def test_sweep_fp64_golden(oracle):
    g = load_golden("sweep_fp64.npz")
    for k, (m, n, p, q) in enumerate(g["cases"]):
        x, l, u = g[f"x{k}"], g[f"l{k}"], g[f"u{k}"]
        assert np.array_equal(oracle.sweep(x, l, u, super_entry_shape=(p, q)), g[f"z_round{k}"]), (m, n, p, q)
        z = oracle.sweep(x, l, u, kind=oracle.Q_ABSMAX, super_entry_shape=(p, q), qmin=-2, qmax=1, half=oracle.BF16)
        assert np.array_equal(z, g[f"z_absmax{k}"]), (m, n, p, q)


def test_sweep_batched_golden(oracle):
    g = load_golden("sweep_batched_fp64.npz")
    for k in range(int(g["count"])):
        z = oracle.sweep_batched(g[f"x{k}"], g[f"l{k}"], g[f"u{k}"], kind=oracle.Q_AFFINE, scale=g[f"scale{k}"],
                                 zero_point=np.zeros((1, 1)))
        assert np.array_equal(z, g[f"z{k}"])


def test_quartic_reference_64(oracle):
    g = load_golden("quartic_64_fp64.npz")
    z = oracle.sweep(g["x"], g["l"], g["u"], kind=oracle.Q_AFFINE, scale=g["scale"], zero_point=np.zeros((64, 64)),
                     qmin=float(g["qmin"]), qmax=float(g["qmax"]))
    assert np.array_equal(z, g["z"])


def test_config0_fp32(oracle):
    for n in (64, 256):
        g = load_golden(f"config0_{n}_fp32.npz")
        scale = np.broadcast_to(g["scale"], (n, n))
        zero = np.zeros((n, n), dtype=np.float32)
        z = oracle.sweep(g["w"], g["l"], g["u"], kind=oracle.Q_AFFINE, scale=scale, zero_point=zero, qmin=-8, qmax=7)
        assert np.array_equal(z, g["z"])
        z1 = oracle.sweep(g["w"], np.eye(n, dtype=np.float32), g["u"], kind=oracle.Q_AFFINE, scale=scale, zero_point=zero, qmin=-8, qmax=7)
        assert np.array_equal(z1, g["z_one_sided"])
        # teacher-forced replay reproduces the same pre-rounding values
        zf, y_pre = oracle.sweep(g["w"], g["l"], g["u"], kind=oracle.Q_FORCED, forced_z=g["z"], return_y_pre=True)
        assert np.array_equal(zf, g["z"])
        assert np.array_equal(oracle.affine_quantize(y_pre, scale, zero, -8, 7), g["z"])


def test_trellis_golden(oracle):
    g = load_golden("trellis.npz")
    for k in range(int(g["count"])):
        for tb in (0, 1):
            values, states = oracle.trellis_quantize(g[f"x{k}"], g[f"table{k}"], int(g[f"K{k}"]), bool(tb))
            assert np.array_equal(values, g[f"values{k}_{tb}"]) and np.array_equal(states, g[f"states{k}_{tb}"]), (k, tb)
    codes = {"hyb": oracle.hyb_from_tlut(g["tlut"]), "one_mad": oracle.one_mad(), "three_inst": oracle.three_inst()}
    for name, table in codes.items():
        digest = np.frombuffer(hashlib.sha256(np.ascontiguousarray(table).tobytes()).digest(), dtype=np.uint8)
        assert np.array_equal(digest, g[f"sha_{name}"]), name
        assert np.array_equal(table[:64], g[f"head_{name}"])
    for name, Ks in (("hyb", (2, 3, 4)), ("one_mad", (2, 4)), ("three_inst", (2,))):
        for K in Ks:
            values, states = oracle.trellis_quantize(g[f"code_x_{name}"], codes[name], K, True)
            assert np.array_equal(values, g[f"code_values_{name}_{K}"]) and np.array_equal(states, g[f"code_states_{name}_{K}"])


def test_trellis_sweep_golden(oracle):
    g = load_golden("trellis_sweep_fp64.npz")
    z = oracle.sweep(g["x"], g["l"], g["u"], kind=oracle.Q_TRELLIS, super_entry_shape=(16, 16), scale=float(g["scale"]),
                     table=g["table"], K=int(g["K"]))
    assert np.array_equal(z, g["z"])


def test_factors_golden(oracle):
    # The reference computes these with LAPACK through torch.linalg: pinned to a tolerance, not bit for bit.
    g = load_golden("factors.npz")
    for n in (1, 7, 64, 200):
        l = oracle.ldl_of_inverse(g[f"g{n}"])
        assert np.allclose(l, g[f"l{n}"], rtol=0, atol=1e-10)
        assert np.array_equal(np.diag(l), np.ones(n)) and np.array_equal(np.triu(l, 1), np.zeros((n, n)))
    for size in (1, 2, 4, 16):
        assert np.allclose(oracle.ldl_of_inverse(g["g48"], size), g[f"l48_{size}"], rtol=0, atol=1e-10)
    l = oracle.ldl_of_inverse(g["g256_f32"])
    assert np.abs(l - g["l256_f32"]).max() < 2e-5
    # property: L^T G L is diagonal (G^{-1} = L Lambda L^T)
    l64 = oracle.ldl_of_inverse(g["g200"])
    d = l64.T @ g["g200"] @ l64
    assert np.abs(d - np.diag(np.diag(d))).max() < 1e-9 * np.abs(np.diag(d)).max()


def test_large_float32_factors_golden(oracle):
    """Heavy-tailed Grams at n = 1024 and 2048: the recipe reproduces the matrices the reference factored, the LAPACK
    restatement equals the reference's float64 rows, and the reference's own float32 rows lie where the fixture says."""
    g = load_golden("factors_fp32_large.npz")
    for n in (1024, 2048):
        gram = oracle.dyadic_gram(n, seed=n)
        assert gram.astype(np.float64).sum() == float(g[f"gram_sum{n}"])  # same bits as when the fixture was made
        rows = g[f"rows{n}"]
        l64 = oracle.ldl_of_inverse_lapack(gram.astype(np.float64))
        assert np.abs(l64[rows] - g[f"l64_{n}"]).max() < 1e-10
        # the stored rows are a sample: their float32-to-float64 distance stays inside the whole factor's
        assert np.abs(g[f"l32_{n}"].astype(np.float64) - g[f"l64_{n}"]).max() <= float(g[f"gap{n}"]) < 3e-6
    small = oracle.dyadic_gram(130, seed=5).astype(np.float64)
    for size in (1, 2, 5):
        assert np.abs(oracle.ldl_of_inverse_lapack(small, size) - oracle.ldl_of_inverse(small, size)).max() < 1e-12


def test_config1_small_golden(oracle):
    """Outliers at 10 sigma and sigma_h = 1 Hessian factors: the oracle's float64 sweep gives the reference's INT4 codes."""
    g = load_golden("config1_small_fp64.npz")
    m, n = 256, 384
    w, gm, hm = oracle.config1_layer(m, n, seed=41)
    assert w.astype(np.float64).sum() == float(g["w_sum"])
    l, u = g["l"].astype(np.float64), g["u"].astype(np.float64)
    assert np.abs(l - oracle.ldl_of_inverse_lapack(gm.astype(np.float64))).max() < 1e-6  # the stored factors are float32-rounded
    scale = np.broadcast_to(g["scale"].astype(np.float64), (m, n))
    assert np.array_equal(oracle.absmax_scale(w, -8, 7, oracle.FP16), g["scale"])
    z = oracle.sweep(w.astype(np.float64), l, u, kind=oracle.Q_AFFINE, scale=scale, zero_point=np.zeros((m, n)), qmin=-8, qmax=7)
    assert np.array_equal(np.rint(z / scale).astype(np.int8), g["codes"])
    assert np.abs(g["codes"]).max() <= 8 and (g["codes"] == -8).any()


def test_d_sided_golden(oracle):
    g = load_golden("d_sided_fp64.npz")
    for k in range(int(g["count"])):
        x = g[f"x{k}"]
        factors = [g[f"l{k}_{d}"] for d in range(x.ndim)]
        assert np.array_equal(oracle.alg4(x, factors), g[f"z{k}"])
    # a 3-factor problem equals the two-sided sweep on the row-major reshape with a Kronecker row factor
    k = 3
    x = g[f"x{k}"]
    l1, l2, l3 = (g[f"l{k}_{d}"] for d in range(3))
    z2 = oracle.sweep(x.reshape(x.shape[0] * x.shape[1], x.shape[2]), np.kron(l1, l2), l3.T.copy())
    assert np.array_equal(z2.reshape(x.shape), g[f"z{k}"])


def test_packed_codes_known_answers(oracle):
    """The packing is this library's own format: pinned by hand-computed bytes and by the round trip."""
    scale = np.full((1, 4), 0.5, dtype=np.float32)
    z = (np.array([[1, 2, 3, 4]], dtype=np.float32) - 8) * scale            # codes 1..4 with qmin = -8
    assert oracle.pack_codes(z, scale, 0.0, -8, 4).tolist() == [[0x21, 0x43]]
    codes3 = np.array([[1, 2, 3, 4, 5, 6, 7, 0, 5]])                           # nine 3-bit fields: 27 bits -> 4 bytes
    value = sum(int(c) << (3 * j) for j, c in enumerate(codes3[0]))
    z3 = (codes3.astype(np.float64) - 2.0) * 0.25                              # zero point 2
    packed = oracle.pack_codes(z3, 0.25, 2.0, 0, 3)
    assert packed.tolist() == [[(value >> (8 * b)) & 0xFF for b in range(4)]]
    assert np.array_equal(oracle.unpack_codes(packed, 0.25, 2.0, 0, 3, 9, np.float64), z3)
    rng = np.random.default_rng(0)
    z = (rng.integers(0, 32, (7, 21)) * 0.125).astype(np.float32)
    assert np.array_equal(oracle.unpack_codes(oracle.pack_codes(z, 0.125, 0.0, 0, 5), 0.125, 0.0, 0, 5, 21), z)


def test_trellis_paths_known_answers(oracle):
    """The stored form of a trellis path is this library's own format: pinned by a hand-computed byte and by the round
    trip through the states of the golden searches (tail-biting strings are read circularly, others carry a header)."""
    # L = 4, one bit per step, not tail-biting: header 101 (upper bits of 1011), then the low bit of 1011, 0110, 1101
    assert oracle.trellis_pack(np.array([[0b1011, 0b0110, 0b1101]]), 4, 1, 1, False).tolist() == [[0b101101]]
    assert oracle.trellis_unpack(np.array([[0b101101]], dtype=np.uint8), 3, 4, 1, 1, False).tolist() == [[0b1011, 0b0110, 0b1101]]
    g = load_golden("trellis.npz")
    checked = 0
    for k in range(int(g["count"])):
        table, K = g[f"table{k}"], int(g[f"K{k}"])
        L, V = table.shape[0].bit_length() - 1, table.shape[1]
        for tail in (0, 1):
            states = g[f"states{k}_{tail}"]
            steps = states.shape[-1]
            if tail and steps * K * V < L:
                continue  # a tail-biting string shorter than one state does not determine it
            codes = oracle.trellis_pack(states, L, K, V, bool(tail))
            assert codes.shape[-1] == ((0 if tail else L - K * V) + steps * K * V + 7) // 8
            assert np.array_equal(oracle.trellis_unpack(codes, steps, L, K, V, bool(tail)), states)
            checked += 1
    assert checked >= 6
