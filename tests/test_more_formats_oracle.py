"""The GGML formats beyond Q4_0 / Q8_0 / Q4_K / Q6_K on the CPU: the C restatement (oracle/xnq_oracle_more.c) against an
independent numpy reading of the reference's block layouts and formulas (k_quants.rs:100-186, 307-610, 834-878, 880-1316,
1507-1722), and its own internal consistency (dot == dot of to_float with the dequantized activation blocks)."""
import numpy as np
import pytest

from oracle import oracle as O
from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

FORMATS = [D.Q4_1, D.Q5_0, D.Q5_1, D.Q2K, D.Q3K, D.Q5K]


@pytest.fixture(scope="module", autouse=True)
def _build():
    O.build()


def _f16(b):
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32).reshape(b.shape[:-1])


def _scale_min_k4(sc12):
    """utils.rs:53-63 for all eight sub-blocks of [..., 12] packed bytes."""
    q = sc12.astype(np.int32)
    sc = np.empty(q.shape[:-1] + (8,), np.int32); mn = np.empty_like(sc)
    for j in range(8):
        if j < 4:
            sc[..., j], mn[..., j] = q[..., j] & 63, q[..., j + 4] & 63
        else:
            sc[..., j] = (q[..., j + 4] & 0xF) | ((q[..., j - 4] >> 6) << 4)
            mn[..., j] = (q[..., j + 4] >> 4) | ((q[..., j] >> 6) << 4)
    return sc, mn


def numpy_to_float(dt, blocks, nelem):
    """Whole-array numpy reading of to_float, written from the struct definitions, not from the C file."""
    b = blocks.reshape(-1, dt.type_size)
    nb = b.shape[0]
    out = np.empty((nb, dt.block_size), np.float32)
    if dt in (D.Q4_1, D.Q5_0, D.Q5_1):
        has_m = dt != D.Q5_0
        five = dt != D.Q4_1
        d = _f16(b[:, 0:2])
        m = _f16(b[:, 2:4]) if has_m else np.zeros(nb, np.float32)
        o = 4 if has_m else 2
        qs = b[:, o + (4 if five else 0):o + (4 if five else 0) + 16].astype(np.int32)
        lo, hi = qs & 0xF, qs >> 4
        if five:
            qh = b[:, o:o + 4].copy().view("<u4").reshape(nb).astype(np.int64)
            j = np.arange(16)
            lo = lo | ((((qh[:, None] >> j) << 4) & 0x10).astype(np.int32))
            hi = hi | (((qh[:, None] >> (j + 12)) & 0x10).astype(np.int32))
        codes = np.concatenate([lo, hi], 1)
        if dt == D.Q5_0:
            out[:] = (codes - 16).astype(np.float32) * d[:, None]
        else:
            out[:] = codes.astype(np.float32) * d[:, None] + m[:, None]
    elif dt == D.Q2K:
        scales, qs, d, dmin = b[:, 0:16].astype(np.int32), b[:, 16:80].astype(np.int32), _f16(b[:, 80:82]), _f16(b[:, 82:84])
        for half in range(2):
            for sh in range(4):
                for part in range(2):
                    sc = scales[:, 8 * half + 2 * sh + part]
                    dl = d * (sc & 0xF).astype(np.float32); ml = dmin * (sc >> 4).astype(np.float32)
                    q = (qs[:, 32 * half + 16 * part:32 * half + 16 * part + 16] >> (2 * sh)) & 3
                    out[:, 128 * half + 32 * sh + 16 * part:128 * half + 32 * sh + 16 * part + 16] = dl[:, None] * q.astype(np.float32) - ml[:, None]
    elif dt == D.Q3K:
        hmask, qs, sc12, d = b[:, 0:32].astype(np.int32), b[:, 32:96].astype(np.int32), b[:, 96:108], _f16(b[:, 108:110])
        a = sc12.copy().view("<u4").reshape(nb, 3).astype(np.int64)
        k1, k2 = 0x03030303, 0x0f0f0f0f
        aux = np.stack([(a[:, 0] & k2) | ((a[:, 2] & k1) << 4), (a[:, 1] & k2) | (((a[:, 2] >> 2) & k1) << 4),
                        ((a[:, 0] >> 4) & k2) | (((a[:, 2] >> 4) & k1) << 4), ((a[:, 1] >> 4) & k2) | (((a[:, 2] >> 6) & k1) << 4)], 1)
        scales = np.stack([(aux[:, w] >> (8 * byte)) & 0xff for w in range(4) for byte in range(4)], 1).astype(np.uint8).view(np.int8).astype(np.float32)
        for half in range(2):
            for sh in range(4):
                bit = 1 << (4 * half + sh)
                for part in range(2):
                    sl = slice(16 * part, 16 * part + 16)
                    q = ((qs[:, 32 * half:32 * half + 32][:, sl] >> (2 * sh)) & 3) - np.where(hmask[:, sl] & bit, 0, 4)
                    dl = d * (scales[:, 8 * half + 2 * sh + part] - np.float32(32.0))
                    o = 128 * half + 32 * sh + 16 * part
                    out[:, o:o + 16] = dl[:, None] * q.astype(np.float32)
    elif dt == D.Q5K:
        d, dmin, qh, qs = _f16(b[:, 0:2]), _f16(b[:, 2:4]), b[:, 16:48].astype(np.int32), b[:, 48:176].astype(np.int32)
        sc, mn = _scale_min_k4(b[:, 4:16])
        for c in range(4):
            ql = qs[:, 32 * c:32 * c + 32]
            for hi in range(2):
                q = ((ql >> 4) if hi else (ql & 0xF)) + np.where(qh & (1 << (2 * c + hi)), 16, 0)
                d1 = d * sc[:, 2 * c + hi].astype(np.float32); m1 = dmin * mn[:, 2 * c + hi].astype(np.float32)
                out[:, 64 * c + 32 * hi:64 * c + 32 * hi + 32] = d1[:, None] * q.astype(np.float32) - m1[:, None]
    return out.reshape(-1)[:nelem]


@pytest.mark.parametrize("dt", FORMATS)
def test_geometry_matches_the_reference_structs(dt):
    sizes = {D.Q4_1: (20, 32), D.Q5_0: (22, 32), D.Q5_1: (24, 32), D.Q8_1: (36, 32), D.Q2K: (84, 256), D.Q3K: (110, 256), D.Q5K: (176, 256)}
    for t, (ts, bs) in sizes.items():
        assert (O.type_size(int(t)), O.block_size(int(t))) == (ts, bs) == (t.type_size, t.block_size)
    assert O.lib().xnqo_vec_dot_type(int(dt)) == int(dt.vec_dot_type)


@pytest.mark.parametrize("dt", FORMATS)
def test_to_float_against_a_numpy_reading_of_the_layout(dt):
    n, k = 6, 1024
    w = synth.make_weight(dt, n, k, seed=3)
    got = O.to_float(int(dt), w, n * k)
    want = numpy_to_float(dt, w, n * k)
    assert np.array_equal(got, want), float(np.abs(got - want).max())


@pytest.mark.parametrize("dt", FORMATS)
def test_dot_equals_the_f64_dot_of_the_dequantized_operands(dt):
    """The reference's own way of checking a quantized dot (k_quants.rs:2162-2184): an f64 dot of both operands as the
    formats define their values. Activation values: Q8_0 q*d; Q8_K q*d; Q8_1 q*d with the offset term m*s taken as written."""
    n, k, m = 5, 1024, 3
    w = synth.make_weight(dt, n, k, seed=4)
    x = synth.make_activation(m, k, seed=5)
    y = O.matmul(int(dt), x, w, n)
    wf = O.to_float(int(dt), w, n * k).reshape(n, k).astype(np.float64)
    adt = dt.vec_dot_type
    ref = np.empty((m, n))
    for r in range(m):
        blocks = O.from_float(int(adt), x[r]).reshape(-1, adt.type_size)
        if adt == D.Q8K:
            a = (blocks[:, 4:260].copy().view(np.int8).astype(np.float64) * blocks[:, 0:4].copy().view(np.float32).astype(np.float64)).reshape(-1)
            ref[r] = wf @ a
        elif adt == D.Q8_0:
            a = (blocks[:, 2:34].copy().view(np.int8).astype(np.float64) * _f16(blocks[:, 0:2]).astype(np.float64)[:, None]).reshape(-1)
            ref[r] = wf @ a
        else:   # Q8_1: sum_j (q_w d_w + m_w) q_a d_a, the reference replaces m_w d_a sum(q_a) by m_w * s (s = f16(sum) * d in f16)
            qa = blocks[:, 4:36].copy().view(np.int8).astype(np.float64); da = _f16(blocks[:, 0:2]).astype(np.float64); s = _f16(blocks[:, 2:4]).astype(np.float64)
            wb = w.reshape(n, -1, dt.type_size)
            mw = _f16(wb[:, :, 2:4]).astype(np.float64)
            scaled = (wf.reshape(n, -1, 32) - mw[:, :, None])              # q_w * d_w
            ref[r] = (scaled * (qa * da[:, None])[None]).sum((1, 2)) + (mw * s[None]).sum(1)
    scale = np.maximum(np.abs(ref), 1.0)
    assert (np.abs(y - ref) / scale).max() < 2e-4, (np.abs(y - ref) / scale).max()


def test_q8_1_blocks_against_numpy():
    """BlockQ8_1::from_float (k_quants.rs:847-873) on rows with ties, zeros and a large value."""
    g = np.random.default_rng(6)
    x = g.standard_normal(32 * 40).astype(np.float32)
    x[0:32] = 0
    x[32:64] = np.linspace(-127, 127, 32, dtype=np.float32) * 0.5     # exact halves after scaling
    x[64] = 1e4
    got = O.from_float(int(D.Q8_1), x).reshape(-1, 36)
    xs = x.reshape(-1, 32)
    amax = np.abs(xs).max(1)
    d = (amax / np.float32(127)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1) / d, np.float32(0)).astype(np.float32)
    v = xs * inv[:, None]
    q = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -128, 127).astype(np.int8)   # round half away from zero
    dh = d.astype(np.float16)
    s = (q.astype(np.int32).sum(1).astype(np.float32).astype(np.float16).astype(np.float32) * dh.astype(np.float32)).astype(np.float16)
    assert np.array_equal(got[:, 4:36].view(np.int8), q)
    assert np.array_equal(got[:, 0:2].copy().view(np.float16).reshape(-1), dh)
    assert np.array_equal(got[:, 2:4].copy().view(np.float16).reshape(-1), s)


@pytest.mark.parametrize("dt", [D.Q4_1, D.Q5_0, D.Q5_1])
def test_simple_quantizers_round_trip(dt):
    g = np.random.default_rng(7)
    x = g.standard_normal(32 * 64).astype(np.float32)
    back = O.to_float(int(dt), O.from_float(int(dt), x), x.size)
    rows = x.reshape(-1, 32)
    if dt == D.Q5_0:   # d = max / -16: codes -16..15 times d; the value opposite the extreme one is clamped by a whole step
        step, worst = np.abs(rows).max(1) / 16, 1.01
    else:
        step, worst = (rows.max(1) - rows.min(1)) / (15 if dt == D.Q4_1 else 31), 0.51
    assert (np.abs(back - x).reshape(-1, 32) <= worst * step[:, None] + 2e-3).all()


def test_odd_block_counts_are_refused_like_the_reference():
    for dt in (D.Q4_1, D.Q5_0, D.Q5_1):
        w = synth.make_weight(dt, 2, 96, seed=8)
        with pytest.raises(ValueError):
            O.matmul(int(dt), synth.make_activation(1, 96), w, 2)
