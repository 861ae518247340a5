"""The one part of the reference that builds in this image, its Q8_0 CUDA kernels (oracle/_ref/reduce.cubin, compiled
from xn-core/cuda-kernels/reduce.cu as it is), run here: its dequantization pins the oracle's and the library's Q8_0
block layout bit for bit, and its matmul is checked the way the reference's own test checks it."""
import numpy as np
import pytest
import torch

from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_cuda():
    from oracle import ref_cuda as r
    if not r.available():
        pytest.skip("oracle/_ref/reduce.cubin has not been built (needs the reference checkout at build time)")
    return r


def test_reference_dequant_kernel_equals_oracle_and_library_bit_for_bit(ref_cuda, O):
    from xn_b200 import quantized as Q
    n, k = 96, 1024
    w = synth.make_weight(D.Q8_0, n, k, seed=300, dscale=0.01)
    ref = ref_cuda.RefQ8(w, n, k).dequantize().cpu().numpy()
    want = O.to_float(int(D.Q8_0), w, n * k).reshape(n, k)
    assert np.array_equal(ref.view(np.uint32), want.view(np.uint32))
    ours = Q.QCudaTensor.from_qtensor(Q.QTensor(w, (n, k), D.Q8_0), "cuda:0").dequantize(torch.float32).cpu().numpy()
    assert np.array_equal(ours.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("m", [1, 3, 16])
def test_reference_matmul_kernel_follows_its_own_test_recipe(ref_cuda, O, m):
    # tests/cuda_tests.rs:2223-2255: against a dense product on the dequantized weight, 1e-4 of max(|want|, 1)
    from xn_b200 import quantized as Q
    n, k = 256, 1024
    w = synth.make_weight(D.Q8_0, n, k, seed=301, dscale=0.01)
    x = synth.make_activation(m, k, seed=302)
    r = ref_cuda.RefQ8(w, n, k)
    got = r.matmul_t(torch.from_numpy(x).cuda()).cpu().numpy()
    dense = O.to_float(int(D.Q8_0), w, n * k).reshape(n, k).astype(np.float64)
    want = x.astype(np.float64) @ dense.T
    assert (np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max() < 1e-4
    # this repository's kernel follows the CPU path instead (activations quantized to Q8_0 first): the two differ
    # by that quantization error, a fraction of a percent of the output scale
    ours = Q.QCudaTensor.from_qtensor(Q.QTensor(w, (n, k), D.Q8_0), "cuda:0").matmul_t(torch.from_numpy(x).cuda()).cpu().numpy()
    rms = float(np.sqrt((want ** 2).mean()))
    assert np.abs(ours - want).max() < 3e-2 * rms
