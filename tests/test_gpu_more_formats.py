"""Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K weights and the Q8_1 activation format on the GPU, through the C-ABI, against the CPU
oracle: upload / canonical bytes round trip, to_float bit for bit, the Q8_1 quantizer byte for byte, matmul within the
reference's metric |g - w| <= 2e-3 * max(|w|, 1) for one row, small batches and a prefill-sized batch."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
FORMATS = [D.Q4_1, D.Q5_0, D.Q5_1, D.Q2K, D.Q3K, D.Q5K]


@pytest.fixture(scope="module", autouse=True)
def _init():
    from xn_b200 import quantized
    O.build()
    quantized.init(DEV)


def _upload(dt, n, k, seed=0, **kw):
    from xn_b200 import quantized as Q
    blocks = synth.make_weight(dt, n, k, seed=seed)
    return blocks, Q.QCudaTensor.from_qtensor(Q.QTensor(blocks, (n, k), dt), DEV, **kw)


@pytest.mark.parametrize("dt", FORMATS)
def test_upload_round_trip_and_to_float_bit_exact(dt):
    n, k = 37, 1024
    blocks, w = _upload(dt, n, k, seed=21)
    assert w.dtype() == dt and tuple(w.shape()) == (n, k)
    assert np.array_equal(w.data(), blocks)
    got = w.dequantize(torch.float32).cpu().numpy().reshape(-1)
    want = O.to_float(int(dt), blocks, n * k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    for tdt in (torch.float16, torch.bfloat16):   # narrower outputs are the f32 values rounded once
        got16 = w.dequantize(tdt).float().cpu().numpy().reshape(-1)
        assert np.array_equal(got16, torch.from_numpy(want).to(tdt).float().numpy())


@pytest.mark.parametrize("dt", FORMATS)
@pytest.mark.parametrize("n,k,m", [(64, 256, 1), (333, 1024, 1), (200, 4096, 5), (96, 2048, 16), (130, 512, 40)])
def test_matmul_against_the_oracle(dt, n, k, m):
    blocks, w = _upload(dt, n, k, seed=22)
    x = synth.make_activation(m, k, seed=23)
    got = w.matmul_t(torch.from_numpy(x).to(DEV)).cpu().numpy()
    want = O.matmul(int(dt), x, blocks, n)
    err = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    assert got.shape == (m, n) and err.max() <= 2e-3, (dt.name, n, k, m, float(err.max()))


@pytest.mark.parametrize("xdt", [torch.float32, torch.float16, torch.bfloat16])
def test_q8_1_activation_blocks_byte_exact(xdt):
    from xn_b200.quantized import quantize_act
    g = torch.Generator().manual_seed(24)
    x = torch.randn(7, 512, generator=g)
    x[0] = 0
    x[1, :32] = torch.linspace(-127, 127, 32) * 0.5
    x[2, 5] = 1e4
    xd = x.to(xdt)
    got = quantize_act(xd.to(DEV), D.Q8_1).cpu().numpy()
    want = np.concatenate([O.from_float(int(D.Q8_1), xd[r].float().numpy()) for r in range(x.shape[0])])
    assert np.array_equal(got, want)


def test_half_outputs_sharded_upload_and_error_paths():
    from xn_b200 import quantized as Q
    from xn_b200._lib import XnqError
    dt, n, k = D.Q5K, 64, 512
    blocks, w = _upload(dt, n, k, seed=25)
    x = torch.from_numpy(synth.make_activation(3, k, seed=26)).to(DEV)
    y32 = w.matmul_t(x)
    for tdt in (torch.float16, torch.bfloat16):
        y = w.matmul_t(x.to(tdt))
        assert y.dtype is tdt
        want = torch.from_numpy(O.matmul(int(dt), x.to(tdt).float().cpu().numpy(), blocks, n)).to(DEV)
        assert torch.allclose(y.float(), want, rtol=1e-2, atol=2e-2)
    # an N-shard of two holds half of the rows and computes exactly those columns
    sh = Q.QCudaTensor.from_qtensor(Q.QTensor(blocks, (n, k), dt), DEV, shard_rank=1, shard_count=2)
    assert torch.equal(sh.matmul_t(x), y32[:, n // 2:])
    # the 32-element formats refuse an odd number of blocks, as the reference's dots do
    b96, w96 = _upload(D.Q4_1, 8, 96, seed=27)
    with pytest.raises(XnqError):
        w96.matmul_t(torch.zeros(1, 96, device=DEV))
