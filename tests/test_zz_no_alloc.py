"""The no-allocation entry point, xnq_matmul_t_static, against the regular one and against the CPU oracle.

Some callers cannot give the library a workspace and cannot let it allocate (their own pool owns the
device memory, or they are recording a CUDA graph); for them the scratch is an array inside the
library. This file is collected last on purpose: if it fails, every other test has already run.
It has to pass both on its own in a fresh process and after the rest of the suite."""
import ctypes

import pytest
import torch

from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32 = 0


def _static(L, t, x, y):
    from xn_b200 import _lib
    m = x.shape[0]
    _lib.check(L.xnq_matmul_t_static(t._h, ctypes.c_void_p(x.data_ptr()), F32, m, x.stride(0) if m > 1 else t.k,
                                     ctypes.c_void_p(y.data_ptr()), F32, y.stride(0) if m > 1 else t.n,
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))


@pytest.mark.parametrize("dt", [D.Q4_0, D.Q8_0, D.Q4K, D.Q6K])
def test_static_scratch_entry_matches_regular_entry_twice_in_a_row(dt, O):
    from xn_b200 import _lib, quantized as Q
    Q.init(DEV)
    L = _lib.lib()
    n, k = 333, 2048
    w = synth.make_weight(dt, n, k, seed=300)
    t = Q.QCudaTensor.from_qtensor(Q.QTensor(w, (n, k), dt), DEV)
    for call, m in enumerate((16, 5, 1, 16)):      # a smaller call after a larger one sees stale scratch behind its own rows
        x = torch.from_numpy(synth.make_activation(m, k, seed=301 + call)).to(DEV)
        want = t.matmul_t(x)
        got = torch.full((m, n), float("nan"), device=DEV)
        _static(L, t, x, got)
        torch.cuda.synchronize()
        err = (got - want).abs() / want.abs().clamp(min=1.0)     # the suite's matmul tolerance: 2e-3 of max(|w|, 1)
        assert torch.isfinite(got).all() and err.max().item() <= 2e-3, (dt.name, m, err.max().item())
        oracle = torch.from_numpy(O.matmul(int(dt), x.cpu().numpy(), w, n))   # the checker of record: the CPU restatement
        oerr = (got.cpu() - oracle).abs() / oracle.abs().clamp(min=1.0)
        assert oerr.max().item() <= 2e-3, (dt.name, m, "vs oracle", oerr.max().item())
        got2 = torch.empty((m, n), device=DEV)
        _static(L, t, x, got2)                                   # second call in a row, same input
        torch.cuda.synchronize()
        assert torch.equal(got2, got)


def test_static_scratch_entry_rejects_what_does_not_fit():
    from xn_b200 import _lib, quantized as Q
    Q.init(DEV)
    L = _lib.lib()
    n, k = 2, 131072                                             # one row of 131072 columns needs 160 KiB of scratch
    t = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(D.Q8_0, n, k, seed=310), (n, k), D.Q8_0), DEV)
    x = torch.zeros((1, k), device=DEV)
    y = torch.zeros((1, n), device=DEV)
    rc = L.xnq_matmul_t_static(t._h, ctypes.c_void_p(x.data_ptr()), F32, 1, k, ctypes.c_void_p(y.data_ptr()), F32, n, None)
    assert rc == -5 and b"scratch" in L.xnq_last_error()
    assert tuple(t.matmul_t(x).shape) == (1, n)                  # the regular entry, with a caller-owned workspace, still serves it
    n, k = 8, 32768                                              # 16 rows x 32768: taken three rows at a time, fits
    t = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(D.Q8_0, n, k, seed=311), (n, k), D.Q8_0), DEV)
    x = torch.from_numpy(synth.make_activation(16, k, seed=312)).to(DEV)
    y = torch.empty((16, n), device=DEV)
    _static(L, t, x, y)
    torch.cuda.synchronize()
    want = t.matmul_t(x)
    assert ((y - want).abs() / want.abs().clamp(min=1.0)).max().item() <= 2e-3
    # a long k where the array holds fewer rows than the kernel would take at once: passes of reduced size
    n, k = 64, 14336
    w = synth.make_weight(D.Q4K, n, k, seed=313)
    t4 = Q.QCudaTensor.from_qtensor(Q.QTensor(w, (n, k), D.Q4K), DEV)
    x4 = torch.from_numpy(synth.make_activation(16, k, seed=314)).to(DEV)
    y4 = torch.empty((16, n), device=DEV)
    _static(L, t4, x4, y4)
    torch.cuda.synchronize()
    want4 = t4.matmul_t(x4)
    assert ((y4 - want4).abs() / want4.abs().clamp(min=1.0)).max().item() <= 2e-3
    n, k = 8, 32768
    rc = L.xnq_matmul_t_static(t._h, ctypes.c_void_p(x.data_ptr()), F32, 17, k, ctypes.c_void_p(y.data_ptr()), F32, n, None)
    assert rc == -5 and b"0..16" in L.xnq_last_error()
    assert L.xnq_matmul_t_static(None, None, F32, 1, 32, None, F32, 8, None) == -1
