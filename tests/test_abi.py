"""CPU tests of the drop-in boundary: libxnq.so loads, exports every symbol include/xnq.h declares,
and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import numpy as np
import pytest

from xn_b200 import _lib
from xn_b200.dtypes import GgmlDType as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for f in os.listdir(os.path.join(ROOT, "include")):
        if f.endswith(".h"):
            text = open(os.path.join(ROOT, "include", f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(xnq_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    syms = declared_symbols()
    assert len(syms) >= 14, syms
    for s in syms:
        assert hasattr(L, s), f"{s} is declared in include/ but not exported by libxnq.so"


def test_version_and_geometry():
    L = _lib.lib()
    assert L.xnq_version() == 1
    for dt in (D.Q4_0, D.Q4_1, D.Q5_0, D.Q5_1, D.Q8_0, D.Q8_1, D.Q2K, D.Q3K, D.Q4K, D.Q5K, D.Q6K, D.Q8K):
        assert L.xnq_type_size(int(dt)) == dt.type_size
        assert L.xnq_block_size(int(dt)) == dt.block_size
    assert L.xnq_type_size(4) == -1 and L.xnq_block_size(5) == -1 and L.xnq_type_size(16) == -1  # ids GGML retired or never used here


def _upload(dtype, buf, nbytes, n, k, rank=0, count=1):
    out = ctypes.c_void_p()
    rc = _lib.lib().xnq_weight_upload(dtype, buf, nbytes, n, k, rank, count, None, ctypes.byref(out))
    return rc, _lib.lib().xnq_last_error().decode()


def test_operand_image_geometry():
    """XNQ_ACT_OPERAND images: 4096 bytes of ticket words, then per 256-k step NP rows of 256 code bytes and NP records of
    32 bytes, NP = 16 / 32 / 64 for up to 16 / 32 / 64 rows; nothing for shapes the integer kernel does not serve."""
    L = _lib.lib()
    for m, np_ in [(1, 16), (2, 16), (16, 16), (17, 32), (32, 32), (33, 64), (64, 64)]:
        for k in (256, 4096, 11008, 14336):
            assert L.xnq_act_operand_bytes(m, k) == 4096 + (k // 256) * np_ * 288, (m, k)
    for m, k in [(0, 4096), (65, 4096), (16, 4100), (16, 0), (-1, 256)]:
        assert L.xnq_act_operand_bytes(m, k) == 0, (m, k)


def test_upload_validation_happens_before_cuda():
    buf = np.zeros(4 * 18, np.uint8)
    p = ctypes.c_void_p(buf.ctypes.data)
    assert _upload(9, p, 72, 4, 32)[0] == -2                      # Q8_1 is an activation format, not a weight format
    assert _upload(4, p, 72, 4, 32)[0] == -2                      # an id GGML retired
    rc, msg = _upload(int(D.Q4_0), p, 72, 4, 33)
    assert rc == -3 and "32-value block" in msg                        # k not a multiple of the block
    rc, msg = _upload(int(D.Q4_0), p, 70, 4, 32)
    assert rc == -5 and "72" in msg                                # byte count mismatch (q8.rs:71-77)
    assert _upload(int(D.Q4_0), p, 72, 4, 32, rank=2, count=2)[0] == -3
    assert _upload(int(D.Q4_0), p, 72, 4, 32, rank=0, count=3)[0] == -3   # n does not divide
    assert _upload(int(D.Q4_0), None, 72, 4, 32)[0] == -1
    assert _lib.lib().xnq_weight_upload(int(D.Q4_0), p, 72, 4, 32, 0, 1, None, None) == -1


def test_null_handles_are_rejected():
    L = _lib.lib()
    assert L.xnq_weight_free(None) == 0
    assert L.xnq_weight_info(None, None, None, None, None, None, None) == -1
    assert L.xnq_weight_dequantize(None, 0, None, None) == -1
    assert L.xnq_weight_canonical_bytes(None, None, 0, None) == -1
    assert L.xnq_matmul_t(None, None, 0, 1, 32, None, 0, 1, None, 0, None) == -1
    assert L.xnq_matmul_workspace_bytes(None, 4) == 0
    assert L.xnq_linear_forward_host(None, None, 1, None, None, None) == -1
    assert L.xnq_quantize_act(2, None, 0, 1, 32, 32, None, None) == -2    # Q4_0 is not an activation format
    assert L.xnq_quantize_act(int(D.Q8K), None, 0, 1, 100, 100, None, None) == -3
    with pytest.raises(_lib.XnqError) as e:
        _lib.check(L.xnq_quantize_act(int(D.Q8_0), None, 0, 1, 32, 32, None, None))
    assert e.value.code == -1


def test_host_mirror_shape_errors_match_reference_messages():
    from xn_b200.quantized import QTensor
    with pytest.raises(ValueError, match="divisible by block size"):
        QTensor(np.zeros(18, np.uint8), (1, 33), D.Q4_0)
    with pytest.raises(ValueError, match="scalar tensor"):
        QTensor(np.zeros(0, np.uint8), (), D.Q4_0)
    with pytest.raises(ValueError, match="wants 72 bytes"):
        QTensor(np.zeros(70, np.uint8), (4, 32), D.Q4_0)
    qt = QTensor(np.zeros(72, np.uint8), (4, 32), D.Q4_0)
    assert qt.rank() == 2 and qt.shape() == (4, 32) and qt.dtype() == D.Q4_0 and qt.storage_size_in_bytes() == 72
