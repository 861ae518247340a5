"""CPU tests of the oracle: the reference's own Q8_0 known-answer recipes, an independent numpy
restatement, agreement between summation orders, and the committed golden vectors."""
import os

import numpy as np
import pytest

from conftest import assert_close_ref
from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

import ref_numpy as R

WEIGHT_TYPES = [D.Q4_0, D.Q8_0, D.Q4K, D.Q6K]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "known_answers.npz")


def test_block_geometry(O):
    # k_quants.rs:98,134,174,196,205 and mod.rs:160-195
    assert [O.type_size(t) for t in (O.Q4_0, O.Q8_0, O.Q4K, O.Q6K, O.Q8K)] == [18, 34, 144, 210, 292]
    assert [O.block_size(t) for t in (O.Q4_0, O.Q8_0, O.Q4K, O.Q6K, O.Q8K)] == [32, 32, 256, 256, 256]
    for t in WEIGHT_TYPES:
        assert t.type_size == O.type_size(int(t)) and t.block_size == O.block_size(int(t))


def test_f16_conversion_matches_ieee(O):
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 4000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, 6.0975e-5, np.inf, -np.inf],
                 np.float32)])
    L = O.lib()
    for v in vals:
        want = np.float32(v).astype(np.float16)
        got = L.xnqo_f32_to_f16(float(v))
        assert got == int(want.view(np.uint16)), (v, got, want.view(np.uint16))
    for h in list(range(0, 0x7c00, 37)) + [0x7bff, 0x0001, 0x03ff, 0x0400, 0x8001, 0xfbff]:
        assert np.float32(L.xnqo_f16_to_f32(h)) == np.array([h], np.uint16).view(np.float16).astype(np.float32)[0]


# ---- the reference's own Q8_0 pins --------------------------------------------------------------
def _q8_0_weights(O, n, k):
    # k_quants.rs:2155-2160 / repack.rs:560-565
    raw = ((np.arange(n * k) * 37 % 211).astype(np.float32) - np.float32(105.0)) / np.float32(64.0)
    return O.from_float(O.Q8_0, raw)


def _lhs(m, k):
    return (((np.arange(m * k) * 53 % 173).astype(np.float32) - np.float32(86.0)) / np.float32(32.0)).reshape(m, k)


@pytest.mark.parametrize("mkn", [(1, 256, 64), (4, 128, 32), (7, 96, 12),                     # k_quants.rs:2191
                                 (1, 768, 3072), (1, 64, 8), (4, 128, 16), (13, 64, 4)])      # repack.rs:570
def test_q8_0_matmul_matches_reference_at_every_pool_size(O, mkn):
    m, k, n = mkn
    w = _q8_0_weights(O, n, k)
    lhs = _lhs(m, k)
    want = O.matmul(O.Q8_0, lhs, w, n, order="f64")
    for threads in (1, 4):
        for order in ("scalar", "avx2"):
            got = O.matmul(O.Q8_0, lhs, w, n, threads=threads, order=order)
            assert_close_ref(got, want, 1e-4, f"{order} threads={threads} {mkn}")


@pytest.mark.parametrize("mkn", [(1, 32, 1), (3, 32, 5), (7, 64, 11), (5, 128, 8), (8, 32, 3), (16, 96, 17), (32, 64, 33)])
def test_sgemm_q8_0_avx_matches_vec_dot(O, mkn):
    # xn-core/tests/quantized_tests.rs:125-218: tolerance 0.0. The reference draws its normals from
    # rand's StdRng, which is not reproducible here; numpy normals of the same distribution stand in.
    m, k, n = mkn
    rng = np.random.default_rng(299792458)
    lhs = rng.standard_normal((m, k), np.float32)
    rhs = rng.standard_normal((n, k), np.float32)
    a = O.from_float(O.Q8_0, lhs)
    b = O.from_float(O.Q8_0, rhs)
    kb = k // 32
    ref = np.empty((m, n), np.float32)
    for i in range(m):
        for j in range(n):
            ref[i, j] = O.vec_dot(O.Q8_0, k, a[i * kb * 34:(i + 1) * kb * 34], b[j * kb * 34:(j + 1) * kb * 34], avx2=True)
    for nth in (1, 3):
        c = np.zeros(m * n, np.float32)
        for ith in range(nth):
            part = O.sgemm_q8_0(m, n, kb, a, b, ith, nth)
            c = np.where(part != 0, part, c)
        assert np.array_equal(c.reshape(n, m).T, ref), mkn


# ---- independent numpy restatement vs the C oracle ------------------------------------------------
@pytest.mark.parametrize("dt", WEIGHT_TYPES)
def test_to_float_matches_numpy_restatement(O, dt):
    n, k = 16, 1024
    w = synth.make_weight(dt, n, k, seed=3)
    got = O.to_float(int(dt), w, n * k)
    want = R.TO_FLOAT[int(dt)](w, n * k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _tricky_activations(m, k, seed):
    x = synth.make_activation(m, k, seed=seed)
    x[0, :32] = 0.0
    if m > 1:
        x[1, :] = 0.0
        x[1, 5] = 1e-30
    if m > 2:
        x[2, 7], x[2, min(200, k - 1)] = 3.25, -3.25   # |x| tie: the first one sets the Q8_K scale's sign
        x[2, :256] = np.clip(x[2, :256], -3.25, 3.25)
    if m > 3:
        x[3] = np.round(x[3] * 4) / 8             # many exact .5 products: round half away from zero
    return x


def test_activation_quantizers_match_numpy_restatement(O):
    x = _tricky_activations(6, 1024, 11)
    assert np.array_equal(O.from_float(O.Q8_0, x), R.from_float_q8_0(x))
    assert np.array_equal(O.from_float(O.Q8K, x), R.from_float_q8k(x))


def test_q8k_zero_block_leaves_bsums_zero(O):
    x = np.zeros(256, np.float32)
    assert not O.from_float(O.Q8K, x).any()


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
def test_summation_orders_agree(O, dt):
    m, k, n = 3, 2048, 96
    w = synth.make_weight(dt, n, k, seed=5)
    x = synth.make_activation(m, k, seed=5)
    f64 = O.matmul(int(dt), x, w, n, order="f64")
    scalar = O.matmul(int(dt), x, w, n, order="scalar")
    avx = O.matmul(int(dt), x, w, n, order="avx2", threads=3)
    assert_close_ref(scalar, f64, 1e-4, f"{dt.name} scalar vs f64")
    assert_close_ref(avx, f64, 1e-4, f"{dt.name} avx2 vs f64")
    assert_close_ref(avx, scalar, 1e-4, f"{dt.name} avx2 vs scalar")


@pytest.mark.parametrize("dt,tol", [(D.Q4_0, 0.14), (D.Q8_0, 0.009), (D.Q4K, 0.09), (D.Q6K, 0.025)])
def test_weight_quantizer_round_trip(O, dt, tol):
    # quantize -> dequantize stays within the format's step (the reference checks q8_0 at 1e-2 of
    # max(|w|,1): xn-core/tests/cuda_tests.rs:2236); inputs N(0,1)
    x = synth.make_activation(8, 1024, seed=13)
    back = O.to_float(int(dt), O.from_float(int(dt), x), x.size).reshape(x.shape)
    err = np.abs(back - x).max() / np.abs(x).max()
    assert err < tol, (dt.name, err)


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
def test_sharded_rows_concatenate_exactly(O, dt):
    m, k, n = 2, 512, 64
    w = synth.make_weight(dt, n, k, seed=9)
    x = synth.make_activation(m, k, seed=9)
    full = O.matmul(int(dt), x, w, n)
    rb = dt.row_bytes(k)
    for g in (2, 4, 8):
        parts = [O.matmul(int(dt), x, w[r * (n // g) * rb:(r + 1) * (n // g) * rb], n // g) for r in range(g)]
        assert np.array_equal(np.concatenate(parts, 1), full)
        assert np.array_equal(synth.make_weight(dt, n, k, seed=9, rows=(n // g, 2 * n // g)), w[(n // g) * rb:(2 * n // g) * rb])


def test_edge_shapes(O):
    for dt in WEIGHT_TYPES:
        k = dt.block_size
        w = synth.make_weight(dt, 1, k, seed=1)
        x = synth.make_activation(1, k, seed=1)
        y = O.matmul(int(dt), x, w, 1)
        assert y.shape == (1, 1) and np.isfinite(y).all()
        assert O.matmul(int(dt), np.zeros((0, k), np.float32), w, 1).shape == (0, 1)
        with pytest.raises(ValueError):
            O.lib()  # keep the binding loaded
            O._check(O.lib().xnqo_to_float(int(dt), None, k + 1, None), "to_float")


def test_golden_vectors(O):
    g = np.load(GOLDEN)
    x = g["x"]
    assert np.array_equal(O.from_float(O.Q8_0, x), g["act_q8_0"])
    assert np.array_equal(O.from_float(O.Q8K, x), g["act_q8k"])
    n, k = 24, 512
    for dt in WEIGHT_TYPES:
        w = g[f"w_{dt.name}"]
        assert np.array_equal(w, synth.make_weight(dt, n, k, seed=7, tensor_id=int(dt))), "generator drifted"
        assert np.array_equal(O.to_float(int(dt), w, n * k).view(np.uint32), g[f"deq_{dt.name}"].view(np.uint32))
        assert np.array_equal(O.matmul(int(dt), x, w, n, threads=1).view(np.uint32), g[f"y_{dt.name}"].view(np.uint32))
        assert np.array_equal(O.from_float(int(dt), g["dense"]), g[f"wq_{dt.name}"])
