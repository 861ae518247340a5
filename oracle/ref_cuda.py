"""TEST INFRASTRUCTURE ONLY. Runs the reference's OWN Q8_0 CUDA kernels (xn-core/cuda-kernels/reduce.cu:847-946,
compiled unmodified for sm_100a into oracle/_ref/reduce.cubin by `make -C oracle ref`) with the reference's
launch geometry (xn-core/src/cuda_backend/q8.rs:137-150): the only piece of the reference that can be built
in this image. Used by tests (to pin the Q8_0 block layout and dequantization against output of the
reference itself) and by `bench.py --impl reference` (its time beside the CPU arm's). Nothing under
xn_b200/ imports this.

The kernels multiply UNQUANTIZED activations with dequantized weights (f32 FMA), unlike the CPU path this
repository reproduces, so their matmul results are compared with a dense product, the way the reference's
own test does (tests/cuda_tests.rs:2223-2255)."""
from __future__ import annotations

import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN = os.path.join(HERE, "_ref", "reduce.cubin")


def available() -> bool:
    return os.path.exists(CUBIN)


def build(ref: str | None = None) -> bool:
    """Compile the reference's kernels where a reference checkout is named (argument or the XN_REFERENCE
    environment variable) and present; returns whether the cubin is there."""
    import subprocess
    ref = ref or os.environ.get("XN_REFERENCE")
    if ref and os.path.exists(os.path.join(ref, "xn-core", "cuda-kernels", "reduce.cu")):
        subprocess.run(["make", "-C", HERE, "ref", f"REF={ref}"], check=True, capture_output=True)
    return available()


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


class RefQ8:
    """The reference's device layout of a Q8_0 weight (q8.rs:78-91: int8 codes [n, k] and f16 scales [n, k/32])
    and its two kernels. Tensors are torch CUDA tensors; launches go on torch's current stream."""

    def __init__(self, blocks: np.ndarray, n: int, k: int, device="cuda:0"):
        import torch
        from cuda.bindings import driver as drv
        self.drv, self.torch, self.n, self.k, self.device = drv, torch, n, k, torch.device(device)
        torch.cuda.init()
        torch.zeros(1, device=self.device)  # make torch's primary context current
        with open(CUBIN, "rb") as f:
            self.module = _check(drv.cuModuleLoadData(f.read()))
        b = np.ascontiguousarray(blocks).view(np.uint8).reshape(n, k // 32, 34)
        self.scales = torch.from_numpy(b[:, :, :2].copy().view(np.float16).reshape(n, k // 32)).to(self.device)
        self.qs = torch.from_numpy(b[:, :, 2:].copy().view(np.int8).reshape(n, k)).to(self.device)

    def _func(self, name: str):
        return _check(self.drv.cuModuleGetFunction(self.module, name.encode()))

    def _launch(self, fn, grid, block, args, arg_types):
        stream = self.torch.cuda.current_stream(self.device).cuda_stream
        _check(self.drv.cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, stream, (tuple(args), tuple(arg_types)), 0))

    def matmul_t(self, x, out=None):
        """`matmul_q8_f32_m{1,2,4,8,16}`: x [m, k] f32, m <= 16 -> [m, n] f32 (q8.rs:116-157)."""
        import ctypes
        m, k = x.shape
        assert k == self.k and m <= 16 and x.dtype == self.torch.float32 and x.is_contiguous()
        mt = 1 << (m - 1).bit_length() if m > 1 else 1
        y = out if out is not None else self.torch.empty((m, self.n), dtype=self.torch.float32, device=self.device)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        self._launch(self._func(f"matmul_q8_f32_m{mt}"), (self.n + 7) // 8, 128,
                     (x.data_ptr(), self.qs.data_ptr(), self.scales.data_ptr(), y.data_ptr(), m, self.n, self.k, self.k),
                     (vp, vp, vp, vp, ci, ci, ci, ci))
        return y

    def dequantize(self):
        """`dequant_q8_f32` (q8.rs:94-113): dense [n, k] f32."""
        import ctypes
        out = self.torch.empty((self.n, self.k), dtype=self.torch.float32, device=self.device)
        numel = self.n * self.k
        self._launch(self._func("dequant_q8_f32"), (numel + 255) // 256, 256, (self.qs.data_ptr(), self.scales.data_ptr(), out.data_ptr(), numel, self.k),
                     (ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int))
        return out
