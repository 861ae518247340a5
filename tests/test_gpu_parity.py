"""GPU parity tests: every call goes through the C ABI (via the ctypes host mirror) and is checked
against the CPU oracle on the same seeded inputs.

Bars: canonical bytes, dequantize and activation quantization are bit-exact; matmul with f32
accumulation is within 2e-3 under the reference's own metric |g-w| <= tol*max(|w|,1)."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_close_ref
from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

pytestmark = pytest.mark.gpu

WEIGHT_TYPES = [D.Q4_0, D.Q8_0, D.Q4K, D.Q6K]
TOL_F32 = 2e-3
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "known_answers.npz")
DEV = "cuda:0"


@pytest.fixture(scope="module")
def Q():
    from xn_b200 import quantized
    quantized.init(DEV)
    return quantized


def _upload(Q, dt, w, n, k, **kw):
    return Q.QCudaTensor.from_qtensor(Q.QTensor(w, (n, k), dt), DEV, **kw)


def test_library_is_loaded_and_device_is_b200(Q):
    from xn_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH)
    assert torch.cuda.get_device_capability(0)[0] == 10


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
@pytest.mark.parametrize("n,kmul", [(1, 1), (7, 3), (33, 8), (130, 16)])
def test_canonical_bytes_round_trip_and_dequantize_bit_exact(Q, O, dt, n, kmul):
    k = dt.block_size * kmul
    w = synth.make_weight(dt, n, k, seed=21)
    t = _upload(Q, dt, w, n, k)
    assert t.shape() == (n, k) and t.dtype() == dt
    assert np.array_equal(t.data(), w), "device layout does not give the canonical GGUF bytes back"
    want = O.to_float(int(dt), w, n * k).reshape(n, k)
    got = t.dequantize(torch.float32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "dequantize is not bit-identical to to_float"
    for td in (torch.float16, torch.bfloat16):
        got_h = t.dequantize(td).float().cpu().numpy()
        assert np.array_equal(got_h, torch.from_numpy(want).to(td).float().numpy())


def _tricky(m, k, seed):
    x = synth.make_activation(m, k, seed=seed)
    x[0, :32] = 0.0
    if m > 1:
        x[1, :] = 0.0
        x[1, 5] = 1e-30
    if m > 2:
        x[2, :256] = np.clip(x[2, :256], -3.25, 3.25)
        x[2, 7], x[2, min(200, k - 1)] = 3.25, -3.25
    if m > 3:
        x[3] = np.round(x[3] * 4) / 8
    return x


@pytest.mark.parametrize("act", [D.Q8_0, D.Q8K])
@pytest.mark.parametrize("m,k", [(1, 256), (5, 1024), (16, 4096), (3, 14336)])
def test_activation_quantizer_bytes_identical(Q, O, act, m, k):
    x = _tricky(m, k, 31 + m)
    want = O.from_float(int(act), x)
    got = Q.quantize_act(torch.from_numpy(x).to(DEV), act).cpu().numpy()
    assert np.array_equal(got, want), f"{act.name} blocks differ at byte {np.flatnonzero(got != want)[:8]}"
    for td in (torch.float16, torch.bfloat16):
        xh = torch.from_numpy(x).to(td)
        want_h = O.from_float(int(act), xh.float().numpy())
        got_h = Q.quantize_act(xh.to(DEV), act).cpu().numpy()
        assert np.array_equal(got_h, want_h), f"{act.name} from {td}"


def test_activation_quantizer_strided_rows(Q, O):
    big = synth.make_activation(4, 1024, seed=5)
    x = torch.from_numpy(big).to(DEV)[:, :512]  # ldx = 1024
    got = Q.quantize_act(x, D.Q8K).cpu().numpy()
    assert np.array_equal(got, O.from_float(O.Q8K, np.ascontiguousarray(big[:, :512])))


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
@pytest.mark.parametrize("m", list(range(1, 17)))
def test_matmul_every_m_up_to_16(Q, O, dt, m):
    n, k = 67, dt.block_size * 6
    w = synth.make_weight(dt, n, k, seed=40)
    x = _tricky(m, k, 40 + m)
    want = O.matmul(int(dt), x, w, n)
    got = _upload(Q, dt, w, n, k).matmul_t(torch.from_numpy(x).to(DEV)).cpu().numpy()
    assert_close_ref(got, want, TOL_F32, f"{dt.name} m={m}")


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
@pytest.mark.parametrize("n,kmul", [(1, 1), (15, 1), (17, 2), (129, 5), (8, 56)])
def test_matmul_edge_shapes(Q, O, dt, n, kmul):
    k = dt.block_size * kmul
    w = synth.make_weight(dt, n, k, seed=50)
    t = _upload(Q, dt, w, n, k)
    for m in (1, 3, 16):
        x = synth.make_activation(m, k, seed=50 + m)
        got = t.matmul_t(torch.from_numpy(x).to(DEV)).cpu().numpy()
        assert_close_ref(got, O.matmul(int(dt), x, w, n), TOL_F32, f"{dt.name} n={n} k={k} m={m}")
    empty = t.matmul_t(torch.zeros((0, k), device=DEV))
    assert tuple(empty.shape) == (0, n)


def test_guard_words_after_output_are_untouched(Q, O):
    dt, n, k, m = D.Q4K, 37, 512, 5
    w = synth.make_weight(dt, n, k, seed=60)
    x = synth.make_activation(m, k, seed=60)
    buf = torch.full((m * n + 64,), 12345.0, device=DEV)
    out = buf[:m * n].view(m, n)
    _upload(Q, dt, w, n, k).matmul_t(torch.from_numpy(x).to(DEV), out=out)
    assert torch.all(buf[m * n:] == 12345.0)
    assert_close_ref(out.cpu().numpy(), O.matmul(int(dt), x, w, n), TOL_F32)


@pytest.mark.parametrize("m", [2, 5, 8, 9, 13, 16])
@pytest.mark.parametrize("n,k", [(70, 256), (130, 4096), (67, 11008), (40, 14336)])
def test_q6k_small_batch_dp4a_shapes(Q, O, m, n, k):
    """Q6_K batches of 2..16 rows stay on the dp4a kernel: from 8 rows on it walks the activation rows once for both weight
    rows of a warp and reads their codes from a swizzled shared-memory image; long rows run in passes of fewer activation
    rows. Ragged row counts, one to 56 super-blocks per row."""
    dt = D.Q6K
    w = synth.make_weight(dt, n, k, seed=300 + m)
    x = _tricky(m, k, 300 + m)
    got = _upload(Q, dt, w, n, k).matmul_t(torch.from_numpy(x).to(DEV)).cpu().numpy()
    assert_close_ref(got, O.matmul(int(dt), x, w, n), TOL_F32, f"Q6K m={m} n={n} k={k}")


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
def test_half_precision_io(Q, O, dt):
    n, k, m = 96, 1024, 4
    w = synth.make_weight(dt, n, k, seed=70)
    t = _upload(Q, dt, w, n, k)
    x = synth.make_activation(m, k, seed=70)
    for td, tol in ((torch.float16, 2e-3), (torch.bfloat16, 1e-2)):
        xh = torch.from_numpy(x).to(td)
        want = O.matmul(int(dt), xh.float().numpy(), w, n)
        got = t.matmul_t(xh.to(DEV))
        assert got.dtype == td
        # output rounding to the 16-bit type dominates: relative to |w|
        err = np.abs(got.float().cpu().numpy() - want) / np.maximum(np.abs(want), 1.0)
        assert err.max() <= tol, (dt.name, td, err.max())


def test_three_d_input_and_bias(Q, O):
    # qlinear_3d_input / qlinear_vs_linear_with_bias shapes: xn-core/tests/quantized_tests.rs:14-118
    dt, n, k = D.Q8_0, 32, 64
    w = synth.make_weight(dt, n, k, seed=80, dscale=0.05)
    x = synth.make_activation(6, k, seed=80).reshape(2, 3, k)
    bias = synth.make_activation(1, n, seed=81)[0]
    lin = Q.QCudaLinear(_upload(Q, dt, w, n, k), torch.from_numpy(bias).to(DEV))
    got = lin.forward(torch.from_numpy(x).to(DEV))
    assert tuple(got.shape) == (2, 3, n)
    want = O.matmul(int(dt), x.reshape(6, k), w, n) + bias
    assert_close_ref(got.cpu().numpy().reshape(6, n), want, TOL_F32)
    with pytest.raises(ValueError, match="only one dimension"):
        lin.forward(torch.zeros(k, device=DEV))
    with pytest.raises(ValueError, match="does not match weight"):
        lin.forward(torch.zeros(2, k + 32, device=DEV))
    host = lin.weight.forward_host(x, bias)
    assert host.shape == (2, 3, n)
    assert_close_ref(host.reshape(6, n), want, TOL_F32)
    # a page-locked result array is written by the kernel itself (no bias, m <= 16); a pageable one is copied into
    # (the Q4_K rows of 11008 values at 16 rows are the shape whose kernel once accumulated into y with atomics: it must not be handed mapped host memory)
    for dt2, n2, k2, m2 in [(D.Q4K, 200, 512, 1), (D.Q6K, 96, 256, 5), (D.Q8_0, 64, 8192, 2), (D.Q4_0, 33, 64, 16), (D.Q4K, 64, 11008, 16), (D.Q5K, 40, 512, 3)]:
        w2 = synth.make_weight(dt2, n2, k2, seed=82)
        x2 = synth.make_activation(m2, k2, seed=83)
        t2 = _upload(Q, dt2, w2, n2, k2)
        want2 = O.matmul(int(dt2), x2, w2, n2)
        pinned = torch.full((m2, n2), float("nan"), dtype=torch.float32).pin_memory()
        got_pinned = t2.forward_host(x2, out=pinned.numpy())
        assert got_pinned is not None and not np.isnan(pinned.numpy()).any()
        assert_close_ref(pinned.numpy(), want2, TOL_F32)
        pageable = np.full((m2, n2), np.nan, np.float32)
        t2.forward_host(x2, out=pageable)
        assert np.array_equal(pageable, pinned.numpy())


def test_q8_0_reference_known_answer_recipe_on_gpu(Q, O):
    # k_quants.rs:2155-2210: closed-form inputs, f64 dot of the quantized operands, 1e-4
    for (m, k, n) in [(1, 256, 64), (4, 128, 32), (7, 96, 12), (13, 64, 4)]:
        raw = ((np.arange(n * k) * 37 % 211).astype(np.float32) - np.float32(105.0)) / np.float32(64.0)
        w = O.from_float(O.Q8_0, raw)
        lhs = (((np.arange(m * k) * 53 % 173).astype(np.float32) - np.float32(86.0)) / np.float32(32.0)).reshape(m, k)
        want = O.matmul(O.Q8_0, lhs, w, n, order="f64")
        got = _upload(Q, D.Q8_0, w, n, k).matmul_t(torch.from_numpy(lhs).to(DEV)).cpu().numpy()
        assert_close_ref(got, want, 1e-4, f"q8_0 {(m, k, n)}")


def test_golden_vectors_without_oracle(Q):
    g = np.load(GOLDEN)
    x = torch.from_numpy(g["x"]).to(DEV)
    assert np.array_equal(Q.quantize_act(x, D.Q8_0).cpu().numpy(), g["act_q8_0"])
    assert np.array_equal(Q.quantize_act(x, D.Q8K).cpu().numpy(), g["act_q8k"])
    n, k = 24, 512
    for dt in WEIGHT_TYPES:
        for key in (f"w_{dt.name}", f"wq_{dt.name}"):
            t = _upload(Q, dt, g[key], n, k)
            assert np.array_equal(t.data(), g[key])
        t = _upload(Q, dt, g[f"w_{dt.name}"], n, k)
        assert np.array_equal(t.dequantize().cpu().numpy().reshape(-1).view(np.uint32), g[f"deq_{dt.name}"].view(np.uint32))
        assert_close_ref(t.matmul_t(x).cpu().numpy(), g[f"y_{dt.name}"], TOL_F32, dt.name)


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
def test_sharded_upload_concatenates_to_unsharded(Q, O, dt):
    """Row shards hold exactly the unsharded tensor's rows. One activation row: every output is one warp's dot in a fixed
    order, so the shards' results are the unsharded ones bit for bit. Several rows: the tensor-core kernel cuts k between
    SMs according to the launch's size, so the f32 grouping (not the integers) differs between a shard and the whole:
    equal within the matmul tolerance, and each launch on its own reproducible."""
    n, k = 64, 1024
    w = synth.make_weight(dt, n, k, seed=90)
    whole = _upload(Q, dt, w, n, k)
    for m in (1, 3):
        x = torch.from_numpy(synth.make_activation(m, k, seed=90)).to(DEV)
        full = whole.matmul_t(x)
        assert torch.equal(whole.matmul_t(x), full), "same launch, same bits"
        for g in (2, 4, 8):
            parts = [_upload(Q, dt, w, n, k, shard_rank=r, shard_count=g) for r in range(g)]
            assert [p.row0 for p in parts] == [r * n // g for r in range(g)] and all(p.n_total == n for p in parts)
            cat = torch.cat([p.matmul_t(x) for p in parts], 1)
            if m == 1:
                assert torch.equal(cat, full)
            else:
                assert_close_ref(cat.cpu().numpy(), full.cpu().numpy(), TOL_F32, f"{dt.name} {g} shards")
            assert np.array_equal(np.concatenate([p.data() for p in parts]), w)


# ---- the benchmark configurations at full size ---------------------------------------------------
FULL = [
    ("C1", D.Q4_0, 4096, 4096, (1,)),
    ("C2", D.Q8_0, 11008, 4096, (1, 16)),
    ("C3", D.Q4K, 14336, 4096, (1, 4, 16)),
    ("C4", D.Q6K, 128256, 4096, (1,)),
    # one whole layer of the 7B decoder of configuration 5 (fused q/k/v, o, fused gate/up, down) and its Q6_K LM head
    ("qkv_proj", D.Q4K, 6144, 4096, (1, 16)),
    ("o_proj", D.Q4K, 4096, 4096, (1, 16)),
    ("gate_up_proj", D.Q4K, 28672, 4096, (1, 16)),
    ("down_proj", D.Q4K, 4096, 14336, (1, 16)),
    ("lm_head", D.Q6K, 32000, 4096, (1, 16)),
]


@pytest.mark.parametrize("name,dt,n,k,ms", FULL)
def test_full_size_configs_against_oracle(Q, O, name, dt, n, k, ms):
    w = synth.make_weight(dt, n, k, seed=0)
    t = _upload(Q, dt, w, n, k)
    for m in ms:
        x = synth.make_activation(m, k, seed=0)
        got = t.matmul_t(torch.from_numpy(x).to(DEV)).cpu().numpy()
        want = O.matmul(int(dt), x, w, n, threads=O.hw_threads())
        assert_close_ref(got, want, TOL_F32, f"{name} m={m}")
        rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
        assert np.abs(got - want).max() / rms < TOL_F32, f"{name} m={m}: error relative to output rms"


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
def test_full_size_properties_without_oracle(Q, dt):
    """Size-independent properties at benchmark size: a one-hot-per-block activation quantizes
    exactly (codes -128/127, scale |x|/127 or x/-128), so the product must equal the matching
    columns of the dequantized weight summed in f32; and the rows of a stacked weight are
    independent of the rows around them."""
    n, k = 4096, 4096
    w = synth.make_weight(dt, n, k, seed=3)
    t = _upload(Q, dt, w, n, k)
    dense = t.dequantize(torch.float32)
    blk = dt.vec_dot_type.block_size
    x = torch.zeros(2, k, device=DEV)
    cols0 = torch.arange(0, k, blk, device=DEV) + 3
    cols1 = torch.arange(0, k, blk, device=DEV) + (blk - 1)
    x[0, cols0] = 1.0
    x[1, cols1] = -2.0
    got = t.matmul_t(x)
    want = torch.stack([dense[:, cols0].double().sum(1), -2.0 * dense[:, cols1].double().sum(1)]).float()
    err = (got - want).abs() / want.abs().clamp(min=1.0)
    assert err.max().item() < 2e-3, err.max().item()
    rb = dt.row_bytes(k)
    sub = Q.QCudaTensor.from_rows(dt, w[1000 * rb:1512 * rb], n, k, 1000, 512, DEV)
    assert torch.equal(sub.matmul_t(x[:1]), t.matmul_t(x[:1])[:, 1000:1512])      # one row: bit for bit
    sub_err = (sub.matmul_t(x) - got[:, 1000:1512]).abs() / got[:, 1000:1512].abs().clamp(min=1.0)
    assert sub_err.max().item() < 2e-3, sub_err.max().item()                      # several rows: k is cut by launch size


@pytest.mark.parametrize("dt", WEIGHT_TYPES)
@pytest.mark.parametrize("n,k", [(1, 256), (15, 512), (16, 1024), (17, 2048), (1000, 4096), (4096, 4096)])
def test_tma_ring_decode_kernel_matches_oracle_and_plain_kernel(Q, O, dt, n, k):
    """m == 1, k <= 4096 takes the persistent TMA-ring kernel; forcing the plain kernel must give
    results within f32 summation order of it, and both must match the oracle."""
    from xn_b200 import _lib
    L = _lib.lib()
    w = synth.make_weight(dt, n, k, seed=100)
    t = _upload(Q, dt, w, n, k)
    x = _tricky(1, k, 100)
    xd = torch.from_numpy(x).to(DEV)
    want = O.matmul(int(dt), x, w, n)
    try:
        _lib.check(L.xnq_set_option(b"matvec_tma", 1))
        got_tma = t.matmul_t(xd).cpu().numpy()
        _lib.check(L.xnq_set_option(b"matvec_tma", 0))
        got_plain = t.matmul_t(xd).cpu().numpy()
    finally:
        _lib.check(L.xnq_set_option(b"matvec_tma", 1))
    assert_close_ref(got_tma, want, TOL_F32, f"tma {dt.name} n={n} k={k}")
    assert_close_ref(got_plain, want, TOL_F32, f"plain {dt.name} n={n} k={k}")
    assert_close_ref(got_tma, got_plain, 1e-4, "tma vs plain")
    for td in (torch.float16, torch.bfloat16):
        xh = torch.from_numpy(x).to(td)
        want_h = O.matmul(int(dt), xh.float().numpy(), w, n)
        got_h = t.matmul_t(xh.to(DEV)).float().cpu().numpy()
        err = np.abs(got_h - want_h) / np.maximum(np.abs(want_h), 1.0)
        assert err.max() <= (2e-3 if td == torch.float16 else 1e-2)


@pytest.mark.parametrize("m", [2, 8, 16, 17, 32, 33, 48, 64])
@pytest.mark.parametrize("n,k", [(128, 256), (200, 1024), (1000, 4096), (300, 11008)])
def test_q4k_small_batch_folded_scales_match_oracle_and_per_block_kernel(Q, O, m, n, k):
    """Q4_K small batches run with the sub-block scales folded into the weight operand (two unsigned planes,
    one drain per 256 block; option 2 forces it for every batch size, the default takes it for 17..32 rows)
    or, with the option 0, with one accumulator slice per 32 elements. Both are
    exact integer sums followed by the same f32 scaling, so both must meet the reference's bound against the
    oracle, and each other up to f32 summation order."""
    from xn_b200 import _lib
    L = _lib.lib()
    dt = D.Q4K
    w = synth.make_weight(dt, n, k, seed=7 + m)
    t = _upload(Q, dt, w, n, k)
    x = _tricky(m, k, 50 + m)
    xd = torch.from_numpy(x).to(DEV)
    want = O.matmul(int(dt), x, w, n)
    try:
        _lib.check(L.xnq_set_option(b"imma_fold", 2))
        got_fold = t.matmul_t(xd).cpu().numpy()
        _lib.check(L.xnq_set_option(b"imma_fold", 0))
        got_blk = t.matmul_t(xd).cpu().numpy()
    finally:
        _lib.check(L.xnq_set_option(b"imma_fold", 1))
    assert_close_ref(got_fold, want, TOL_F32, f"fold m={m} n={n} k={k}")
    assert_close_ref(got_blk, want, TOL_F32, f"per-block m={m} n={n} k={k}")
    assert_close_ref(got_fold, got_blk, 5e-4, "fold vs per-block")


def test_zz_device_status_is_clean(Q):
    """No bounded wait inside any kernel of this session expired."""
    import ctypes
    from xn_b200 import _lib
    bits = ctypes.c_uint(123)
    _lib.check(_lib.lib().xnq_device_status(ctypes.byref(bits)))
    assert bits.value == 0, f"device status bits {bits.value:#x}"


def test_activation_quantizer_rounding_ties_and_near_ties(Q, O):
    """Rust's f32::round is half away from zero. With a block maximum of 127 (Q8_0: scale 1) or a
    first-largest element of -128 (Q8_K: iscale 1) the products equal the inputs, so exact .5 ties,
    the floats just below .5 and the saturating 127.5 -> 127 case reach the rounding step as written."""
    below_half = np.nextafter(np.float32(0.5), np.float32(0))
    vals = np.array([0.5, 1.5, 2.5, 3.5, -0.5, -1.5, -2.5, 126.5, -126.5, below_half, -below_half, 0.25, -0.75,
                     np.nextafter(np.float32(1.5), np.float32(0)), np.nextafter(np.float32(2.5), np.float32(3)), 63.5, -63.5,
                     100.49999, -100.5, 7.5000005, 1e-8, -1e-8, 0.0, 126.49999, 125.5, -0.0, 31.5, -31.5, 15.5, 8.5, -8.5],
                    np.float32)
    x8 = np.zeros((2, 256), np.float32)
    for r in range(2):
        for b in range(8):
            blk = np.roll(vals, 3 * b + r)[:31]
            x8[r, 32 * b] = 127.0 if (b + r) % 2 == 0 else -127.0
            x8[r, 32 * b + 1:32 * b + 32] = blk
    got = Q.quantize_act(torch.from_numpy(x8).to(DEV), D.Q8_0).cpu().numpy()
    assert np.array_equal(got, O.from_float(O.Q8_0, x8))
    xk = np.zeros((2, 512), np.float32)
    for r in range(2):
        for b in range(2):
            xk[r, 256 * b:256 * b + 256] = np.resize(np.roll(vals, b + 5 * r), 256)
            xk[r, 256 * b + 17] = -128.0
            xk[r, 256 * b + 40] = 127.5      # rounds to 128, clipped to 127
            xk[r, 256 * b + 90] = 128.0      # same magnitude as the maximum but later: must not win
    got = Q.quantize_act(torch.from_numpy(xk).to(DEV), D.Q8K).cpu().numpy()
    want = O.from_float(O.Q8K, xk)
    assert np.array_equal(got, want), np.flatnonzero(got != want)[:10]


@pytest.mark.parametrize("m", [5, 9, 16])
def test_q4k_small_batch_at_large_k_two_staged_halves(Q, O, m):
    """k = 14336 (the 7B down projection): above 8 rows the activation image of the whole k does not fit shared
    memory, each CTA stages one half and the halves meet in the output; f16 output takes two passes of 8 rows."""
    dt, n, k = D.Q4K, 272, 14336
    w = synth.make_weight(dt, n, k, seed=90)
    x = synth.make_activation(m, k, seed=91)
    t = _upload(Q, dt, w, n, k)
    want = O.matmul(int(dt), x, w, n)
    xd = torch.from_numpy(x).to(DEV)
    for rep in range(2):   # the output buffer is reused: the second call must not add onto the first
        out = torch.full((m, n), 7.0, device=DEV)
        got = t.matmul_t(xd, out=out).cpu().numpy()
        assert_close_ref(got, want, TOL_F32)
    # f16 in and out: the oracle sees the same f16-rounded activations; the f16 output rounds at 5e-4 of each value
    x16 = x.astype(np.float16)
    want16 = O.matmul(int(dt), x16.astype(np.float32), w, n)
    got16 = t.matmul_t(torch.from_numpy(x16).to(DEV)).float().cpu().numpy()
    rms = float(np.sqrt((want16 ** 2).mean()))
    assert (np.abs(got16 - want16) / np.maximum(np.abs(want16), rms)).max() < 2e-3
