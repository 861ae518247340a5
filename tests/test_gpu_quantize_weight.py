"""Device weight quantizers against the CPU oracle's from_float: every byte of every block."""
import numpy as np
import pytest
import torch

from xn_b200.dtypes import GgmlDType as D

pytestmark = pytest.mark.gpu

FORMATS = [D.Q4_0, D.Q8_0, D.Q4K, D.Q6K]


@pytest.fixture(scope="module")
def Q():
    from xn_b200 import quantized
    quantized.init(torch.device("cuda", 0))
    return quantized


def _dense(n, k, seed, kind):
    rng = np.random.default_rng(seed)
    if kind == "normal":            # the distribution model weights have
        w = rng.normal(0, 0.02, (n, k))
    elif kind == "wide":            # several orders of magnitude between rows and inside blocks
        w = rng.normal(0, 1, (n, k)) * np.exp(rng.normal(0, 3, (n, 1))) * np.exp(rng.normal(0, 1, (n, k)))
    elif kind == "positive":        # min > 0 paths of make_qkx1_quants
        w = np.abs(rng.normal(0, 1, (n, k))) + 0.5
    elif kind == "negative":
        w = -np.abs(rng.normal(0, 1, (n, k))) - 0.5
    elif kind == "lattice":         # few distinct values: ties in nearest_int and early exits of the searches
        w = rng.integers(-3, 4, (n, k)) * 0.25
    elif kind == "sparse":          # all-zero and constant sub-blocks, single spikes
        w = np.zeros((n, k))
        w[::3, ::17] = rng.normal(0, 1, w[::3, ::17].shape)
        w[1, :64] = 0.75
        w[2, 5] = -1e-30
        w[4, 300:316] = 3.0
    else:
        raise ValueError(kind)
    return np.ascontiguousarray(w, np.float32)


@pytest.mark.parametrize("kind", ["normal", "wide", "positive", "negative", "lattice", "sparse"])
@pytest.mark.parametrize("dt", FORMATS, ids=lambda d: d.name)
def test_device_quantizer_is_byte_identical_to_the_oracle(Q, O, dt, kind):
    n, k = 24, 1024
    w = _dense(n, k, 7 + int(dt), kind)
    want = np.frombuffer(O.from_float(int(dt), w), np.uint8)
    got = Q.quantize_weight(torch.from_numpy(w).cuda(), dt).cpu().numpy()
    assert got.shape == want.shape
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, f"{dt.name}/{kind}: {bad.size} bytes differ, first at {bad[:8]} (block {bad[0] // dt.type_size}, offset {bad[0] % dt.type_size})"


@pytest.mark.parametrize("dt", FORMATS, ids=lambda d: d.name)
def test_from_linear_matches_quantize_then_upload(Q, O, dt):
    """QLinear::from_linear: quantize on the device, keep the blocks there, and multiply; the result equals
    the oracle's matmul on the oracle-quantized weight, and the stored bytes are the oracle's."""
    n, k, m = 96, 512, 3
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    blocks = np.frombuffer(O.from_float(int(dt), w), np.uint8)
    lin = Q.QCudaLinear.from_linear(torch.from_numpy(w).cuda(), dt)
    assert np.array_equal(lin.weight.data(), blocks)
    ref = O.matmul(int(dt), x, blocks, n, threads=2)
    y = lin(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.abs(y - ref).max() <= 2e-3 * max(1.0, float(np.abs(ref).max()))


def test_quantize_weight_rejects_bad_shapes(Q):
    from xn_b200._lib import XnqError
    with pytest.raises(ValueError):
        Q.quantize_weight(torch.zeros((4, 100), device="cuda"), D.Q4K)
    with pytest.raises((ValueError, XnqError)):
        Q.quantize_weight(torch.zeros((4,), device="cuda"), D.Q4_0)
