"""ctypes binding of the CPU oracle (``libxnq_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the benchmark's CPU
baseline leg.  The shipped package never imports it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libxnq_oracle.so")

F32, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2K, Q3K, Q4K, Q5K, Q6K, Q8K = 0, 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (gcc only)."""
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".c", ".h")) or f == "Makefile"]
    stale = force or not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.xnqo_type_size.argtypes = [ci]
        L.xnqo_block_size.argtypes = [ci]
        L.xnqo_vec_dot_type.argtypes = [ci]
        L.xnqo_f32_to_f16.argtypes = [ctypes.c_float]
        L.xnqo_f32_to_f16.restype = ctypes.c_uint16
        L.xnqo_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.xnqo_f16_to_f32.restype = ctypes.c_float
        L.xnqo_to_float.argtypes = [ci, vp, i64, vp]
        L.xnqo_from_float.argtypes = [ci, vp, i64, vp]
        L.xnqo_vec_dot.argtypes = [ci, i64, vp, vp, vp]
        L.xnqo_vec_dot_avx2.argtypes = [ci, i64, vp, vp, vp]
        L.xnqo_matmul.argtypes = [ci, i64, i64, i64, vp, vp, vp, ci]
        L.xnqo_matmul_f64.argtypes = [ci, i64, i64, i64, vp, vp, vp, ci]
        L.xnqo_matmul_avx2.argtypes = [ci, i64, i64, i64, vp, vp, vp, ci]
        L.xnqo_matmul_avx2_prequant.argtypes = [ci, i64, i64, i64, vp, vp, vp, ci]
        L.xnqo_sgemm_q8_0.argtypes = [i64, i64, i64, vp, i64, vp, i64, vp, i64, ci, ci]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"oracle {what} failed with code {rc}")


def type_size(dtype: int) -> int:
    return lib().xnqo_type_size(int(dtype))


def block_size(dtype: int) -> int:
    return lib().xnqo_block_size(int(dtype))


def hw_threads() -> int:
    return lib().xnqo_hw_threads()


def have_avx2() -> bool:
    return bool(lib().xnqo_have_avx2())


def to_float(dtype: int, blocks: np.ndarray, nelem: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
    assert blocks.size == nelem // block_size(dtype) * type_size(dtype), "block byte count"
    out = np.empty(nelem, np.float32)
    _check(lib().xnqo_to_float(int(dtype), _p(blocks), nelem, _p(out)), "to_float")
    return out


def from_float(dtype: int, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    out = np.zeros(x.size // block_size(dtype) * type_size(dtype), np.uint8)
    _check(lib().xnqo_from_float(int(dtype), _p(x), x.size, _p(out)), "from_float")
    return out


def vec_dot(dtype: int, k: int, w_row: np.ndarray, act_row: np.ndarray, avx2: bool = False) -> float:
    out = np.zeros(1, np.float32)
    fn = lib().xnqo_vec_dot_avx2 if avx2 else lib().xnqo_vec_dot
    _check(fn(int(dtype), k, _p(np.ascontiguousarray(w_row)), _p(np.ascontiguousarray(act_row)), _p(out)), "vec_dot")
    return float(out[0])


def matmul(dtype: int, lhs: np.ndarray, rhs_blocks: np.ndarray, n: int, threads: int = 0,
           order: str = "scalar") -> np.ndarray:
    """``lhs @ W^T`` with lhs ``[m, k]`` f32 and W given as canonical blocks of ``[n, k]``.

    order: "scalar" (vec_dot_unopt order; the parity oracle), "avx2" (the order xn's x86 build
    computes in; the timed baseline) or "f64" (exact dot of the quantized operands)."""
    lhs = np.ascontiguousarray(lhs, np.float32)
    m, k = lhs.shape
    rhs = np.ascontiguousarray(rhs_blocks).view(np.uint8).reshape(-1)
    assert rhs.size == n * (k // block_size(dtype)) * type_size(dtype), "weight byte count"
    if order == "f64":
        dst = np.zeros((m, n), np.float64)
        _check(lib().xnqo_matmul_f64(int(dtype), m, k, n, _p(lhs), _p(rhs), _p(dst), threads), "matmul_f64")
        return dst
    dst = np.zeros((m, n), np.float32)
    fn = {"scalar": lib().xnqo_matmul, "avx2": lib().xnqo_matmul_avx2}[order]
    _check(fn(int(dtype), m, k, n, _p(lhs), _p(rhs), _p(dst), threads), f"matmul[{order}]")
    return dst


def matmul_avx2_prequant(dtype: int, m: int, k: int, n: int, lhs_blocks: np.ndarray, rhs_blocks: np.ndarray,
                         dst: np.ndarray, threads: int = 0) -> None:
    _check(lib().xnqo_matmul_avx2_prequant(int(dtype), m, k, n, _p(lhs_blocks), _p(rhs_blocks), _p(dst), threads),
           "matmul_avx2_prequant")


def sgemm_q8_0(m: int, n: int, kblocks: int, a: np.ndarray, b: np.ndarray, ith: int = 0, nth: int = 1) -> np.ndarray:
    """Column-major ``c[m*j + i]`` from a ``[m, k]`` and b ``[n, k]`` Q8_0 blocks (avx.rs:115-164)."""
    c = np.zeros(m * n, np.float32)
    _check(lib().xnqo_sgemm_q8_0(m, n, kblocks, _p(a), kblocks, _p(b), kblocks, _p(c), m, ith, nth), "sgemm_q8_0")
    return c
