"""Host-side mirror of xn-core's quantized operator API, over the xnq C ABI.

Names, argument meaning and error behaviour follow the reference so that its tests read the same
here:

=====================  ==========================================================================
``QTensor``            xn-core/src/quantized/mod.rs:27-340 (host blocks + shape; canonical bytes)
``QCudaTensor``        the device weight; API of ``Q8Tensor`` (cuda_backend/q8.rs:26-157)
``QCudaLinear``        ``Q8Linear`` (q8.rs:160-185) / ``QLinear`` (mod.rs:342-406)
``Q40 Q80 Q4K Q6K``    ``BackendQ`` implementations (lib.rs:141-156; q8.rs:187-224)
=====================  ==========================================================================

torch supplies device memory, streams and tensors; every computation happens in ``libxnq.so``.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import XnqError, check
from .dtypes import GgmlDType

_TORCH_TO_XNQ = {torch.float32: GgmlDType.F32, torch.float16: GgmlDType.F16, torch.bfloat16: GgmlDType.BF16}


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_inited: set[int] = set()
_workspaces: dict[int, list[torch.Tensor]] = {}


def init(device: torch.device | int | str = "cuda:0") -> None:
    """``xnq_init`` for the device (idempotent). Call before capturing a CUDA graph."""
    dev = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx in _inited:
        return
    torch.cuda.init()
    with torch.cuda.device(idx):
        torch.empty(1, device=f"cuda:{idx}")  # make the primary context current on this thread
        check(_lib.lib().xnq_init(idx))
    _inited.add(idx)


class QTensor:
    """Quantized blocks in host memory with a shape (mod.rs:27-340). ``data()`` is canonical GGUF bytes."""

    def __init__(self, data: np.ndarray | bytes, shape: Sequence[int], dtype: GgmlDType):
        dtype = GgmlDType(dtype)
        shape = tuple(int(d) for d in shape)
        if len(shape) == 0:
            raise ValueError(f"scalar tensor cannot be quantized {shape}")  # mod.rs:264-266
        if shape[-1] % dtype.block_size:
            raise ValueError(
                f"quantized tensor must have their last dim divisible by block size {shape} {dtype.block_size}")  # mod.rs:267-272
        buf = np.frombuffer(data, np.uint8) if isinstance(data, (bytes, bytearray, memoryview)) else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        want = int(np.prod(shape)) // dtype.block_size * dtype.type_size
        if buf.size != want:
            raise ValueError(f"{dtype.name} {shape} wants {want} bytes of blocks, got {buf.size}")
        self._data, self._shape, self._dtype = buf, shape, dtype

    @classmethod
    def new(cls, data, shape, dtype) -> "QTensor":
        return cls(data, shape, dtype)

    def dtype(self) -> GgmlDType:
        return self._dtype

    def rank(self) -> int:
        return len(self._shape)

    def shape(self) -> tuple[int, ...]:
        return self._shape

    def storage_size_in_bytes(self) -> int:
        return int(self._data.size)

    def data(self) -> np.ndarray:
        """Canonical on-disk bytes (mod.rs:330-332)."""
        return self._data


class QCudaTensor:
    """A ``(n, k)`` quantized weight (or an N-shard of one) resident on a CUDA device."""

    def __init__(self, handle: int, device: torch.device):
        self._h = ctypes.c_void_p(handle)
        self.device = device
        dt, nt, nl, r0, k, nb = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_size_t()
        check(_lib.lib().xnq_weight_info(self._h, dt, nt, nl, r0, k, nb))
        self._dtype = GgmlDType(dt.value)
        self.n_total, self.n, self.row0, self.k, self.device_bytes = nt.value, nl.value, r0.value, k.value, nb.value
        self._ws: Optional[torch.Tensor] = None

    # -- construction ---------------------------------------------------------------------------
    @classmethod
    def from_qtensor(cls, qt: QTensor, device: torch.device | str = "cuda:0", shard_rank: int = 0,
                     shard_count: int = 1) -> "QCudaTensor":
        """Take GGUF blocks as they are (``Q8Tensor::from_q8_0``, q8.rs:60-85)."""
        device = torch.device(device)
        if not qt.dtype().is_quantized_weight:
            raise ValueError(f"cuda quantized: expected a quantized weight format, got {qt.dtype().name}")
        if qt.rank() != 2:
            raise ValueError(f"cuda quantized: expected a 2-d weight, got shape {qt.shape()}")
        n, k = qt.shape()
        init(device)
        out = ctypes.c_void_p()
        buf = qt.data()
        with torch.cuda.device(device):
            check(_lib.lib().xnq_weight_upload(int(qt.dtype()), ctypes.c_void_p(buf.ctypes.data), buf.size, n, k,
                                               shard_rank, shard_count, _stream_ptr(device), ctypes.byref(out)))
        return cls(out.value, device)

    @classmethod
    def from_dense(cls, weight: torch.Tensor, dtype: GgmlDType, shard_rank: int = 0, shard_count: int = 1) -> "QCudaTensor":
        """Quantize a dense ``[n, k]`` device tensor with the reference's quantizer for ``dtype`` (run on the
        GPU, same bits) and keep the blocks on the device: ``QTensor::quantize_f32`` + ``from_qtensor``
        (mod.rs:290-297, q8.rs:218-223) without the trip through host memory."""
        dtype = GgmlDType(dtype)
        if weight.dim() != 2:
            raise ValueError(f"cuda quantized: expected a 2-d weight, got shape {tuple(weight.shape)}")
        n, k = weight.shape
        blocks = quantize_weight(weight, dtype)
        out = ctypes.c_void_p()
        with torch.cuda.device(weight.device):
            check(_lib.lib().xnq_weight_upload(int(dtype), ctypes.c_void_p(blocks.data_ptr()), blocks.numel(), n, k,
                                               shard_rank, shard_count, _stream_ptr(weight.device), ctypes.byref(out)))
        return cls(out.value, weight.device)

    @classmethod
    def from_rows(cls, dtype: GgmlDType, blocks: np.ndarray, n_total: int, k: int, row0: int, n_rows: int,
                  device: torch.device | str = "cuda:0") -> "QCudaTensor":
        """Upload rows ``[row0, row0 + n_rows)`` of an ``[n_total, k]`` weight from their own bytes."""
        device = torch.device(device)
        init(device)
        out = ctypes.c_void_p()
        buf = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        with torch.cuda.device(device):
            check(_lib.lib().xnq_weight_upload_rows(int(dtype), ctypes.c_void_p(buf.ctypes.data), buf.size, n_total, k, row0,
                                                    n_rows, _stream_ptr(device), ctypes.byref(out)))
        return cls(out.value, device)

    @classmethod
    def from_device_rows(cls, dtype: GgmlDType, blocks: torch.Tensor, n_total: int, k: int, row0: int, n_rows: int) -> "QCudaTensor":
        """``from_rows`` for canonical blocks that already sit in device memory (a uint8 tensor)."""
        init(blocks.device)
        out = ctypes.c_void_p()
        buf = blocks.contiguous().view(torch.uint8).reshape(-1)
        with torch.cuda.device(blocks.device):
            check(_lib.lib().xnq_weight_upload_rows(int(dtype), ctypes.c_void_p(buf.data_ptr()), buf.numel(), n_total, k, row0,
                                                    n_rows, _stream_ptr(blocks.device), ctypes.byref(out)))
        return cls(out.value, blocks.device)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.lib().xnq_weight_free(h)
            except Exception:
                pass

    # -- queries --------------------------------------------------------------------------------
    def dtype(self) -> GgmlDType:
        return self._dtype

    def shape(self) -> tuple[int, int]:
        """Shape of the rows held on this device."""
        return (self.n, self.k)

    def data(self) -> np.ndarray:
        """Canonical GGUF bytes of the held rows, back on the host."""
        out = np.empty(self.n * self._dtype.row_bytes(self.k), np.uint8)
        with torch.cuda.device(self.device):
            check(_lib.lib().xnq_weight_canonical_bytes(self._h, ctypes.c_void_p(out.ctypes.data), out.size, _stream_ptr(self.device)))
        return out

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """The weight as a dense ``(n, k)`` matrix (q8.rs:94-113)."""
        out = torch.empty((self.n, self.k), dtype=dtype, device=self.device)
        with torch.cuda.device(self.device):
            check(_lib.lib().xnq_weight_dequantize(self._h, int(_TORCH_TO_XNQ[dtype]), ctypes.c_void_p(out.data_ptr()), _stream_ptr(self.device)))
        return out

    # -- compute --------------------------------------------------------------------------------
    def workspace(self, m: int) -> torch.Tensor:
        """Scratch for ``m`` activation rows. All weights of a device share one buffer (the reference's device
        has a single stream, cuda_backend/mod.rs:141-167, so calls never overlap); it only ever grows, and
        outgrown buffers stay alive because a captured graph may still point at them."""
        need = _lib.lib().xnq_matmul_workspace_bytes(self._h, m)
        pool = _workspaces.setdefault(self.device.index or 0, [])
        if not pool or pool[-1].numel() < need:
            pool.append(torch.empty(max(need, 256), dtype=torch.uint8, device=self.device))
        return pool[-1]

    def hint_next(self) -> None:
        """Names this weight as the one the calling thread multiplies after its next one-row matmul: that matmul's kernel
        asks for these bytes to be brought into L2 while it finishes (xnq_hint_next_weight)."""
        check(_lib.lib().xnq_hint_next_weight(self._h))

    def supports_normed(self) -> bool:
        """Whether :meth:`matvec_normed` serves this weight (rows of at most 4096 values on the one-row kernel)."""
        return self._dtype.has_fast_kernels and self.k <= 4096 and self.k % 256 == 0

    def matvec_normed(self, x_in: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float, x_out: torch.Tensor,
                      out: torch.Tensor, await_comm=None) -> torch.Tensor:
        """One row: ``x_out = x_in + delta`` (``delta`` may hold several summands side by side, or be None), then
        ``out = self . quantize(rmsnorm(x_out) * norm_weight)`` in ONE launch of the one-row kernel; bit for bit what
        ``add_rmsnorm`` with an activation image followed by :meth:`matmul_t` gives (xnq_matvec_normed; the rms_norm +
        linear pairs of llama.rs:145-216). ``x_out`` must be another buffer than ``x_in``. ``await_comm``: the ``PeerGather``
        whose slot holds ``delta`` when that gather was issued in deferred mode (the kernel then awaits the peers itself)."""
        for t in (x_in, delta, norm_weight, x_out):
            if t is not None and (t.dtype is not torch.float32 or not t.is_contiguous() or t.device != self.device):
                raise ValueError("matvec_normed: f32 contiguous tensors on the weight's device")
        if x_in.numel() != self.k or x_out.numel() != self.k or norm_weight.numel() != self.k or out.numel() != self.n:
            raise ValueError(f"matvec_normed: shapes do not match weight (n={self.n}, k={self.k})")
        parts = 0 if delta is None else delta.numel() // self.k
        p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
        with torch.cuda.device(self.device):
            check(_lib.lib().xnq_matvec_normed(self._h, p(x_in), p(delta), parts, p(norm_weight), eps, p(x_out), p(out), int(_TORCH_TO_XNQ[out.dtype]),
                                               await_comm._h if await_comm is not None else None, _stream_ptr(self.device)))
        return out

    def matmul_t(self, lhs: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``lhs @ self^T`` with ``lhs`` of shape ``(.., k)``; the result is ``(.., n)`` (q8.rs:116-157)."""
        if hasattr(lhs, "act_dtype"):   # an ActImage: activations quantized ahead of the call
            if lhs.k != self.k or lhs.act_dtype != self._dtype.vec_dot_type:
                raise ValueError(f"cuda quantized matmul: image [{lhs.m}, {lhs.k}] {lhs.act_dtype.name} does not fit weight (k={self.k}, {self._dtype.name})")
            if out is None:
                out = torch.empty((lhs.m, self.n), dtype=torch.float32, device=self.device)
            y = out.view(-1, self.n)
            ws = self.workspace(lhs.m) if lhs.m > 1 else None   # batches go to the tensor-core kernel, which re-lays the image out in scratch
            with torch.cuda.device(self.device):
                check(_lib.lib().xnq_matmul_t(self._h, ctypes.c_void_p(lhs.data_ptr()), _lib.XNQ_ACT_OPERAND if getattr(lhs, "operand", False) else _lib.XNQ_ACT_IMAGE,
                                              lhs.m, 0, ctypes.c_void_p(y.data_ptr()),
                                              int(_TORCH_TO_XNQ[y.dtype]), y.stride(0) if lhs.m > 1 else self.n,
                                              ctypes.c_void_p(ws.data_ptr()) if ws is not None else None, ws.numel() if ws is not None else 0,
                                              _stream_ptr(self.device)))
            return out
        if lhs.shape[-1] != self.k:
            raise ValueError(f"cuda quantized matmul: input {tuple(lhs.shape)} does not match weight (n={self.n}, k={self.k})")
        if lhs.dtype not in _TORCH_TO_XNQ:
            raise ValueError(f"cuda quantized matmul: unsupported activation dtype {lhs.dtype}")
        if lhs.device != self.device:
            raise ValueError(f"cuda quantized matmul: input on {lhs.device}, weight on {self.device}")
        x = lhs.reshape(-1, self.k)
        if x.stride(-1) != 1 or (x.shape[0] > 1 and x.stride(0) < self.k):
            x = x.contiguous()
        m = x.shape[0]
        ldx = x.stride(0) if m > 1 else self.k
        if out is None:
            out = torch.empty(lhs.shape[:-1] + (self.n,), dtype=lhs.dtype, device=self.device)
        y = out.view(-1, self.n)
        ws = self.workspace(m)
        with torch.cuda.device(self.device):
            check(_lib.lib().xnq_matmul_t(self._h, ctypes.c_void_p(x.data_ptr()), int(_TORCH_TO_XNQ[x.dtype]), m, ldx,
                                          ctypes.c_void_p(y.data_ptr()), int(_TORCH_TO_XNQ[y.dtype]), y.stride(0) if m > 1 else self.n,
                                          ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(self.device)))
        return out

    def forward_host(self, x: np.ndarray, bias: Optional[np.ndarray] = None, out: Optional[np.ndarray] = None) -> np.ndarray:
        """``QLinear::forward`` on host arrays (mod.rs:352-384): H2D copy, matmul, optional bias, D2H copy, sync.
        ``out`` may name the result array (for instance the numpy view of a pinned torch tensor, which the
        kernel then writes directly)."""
        x = np.ascontiguousarray(x, np.float32)
        if x.ndim < 2:
            raise ValueError(f"input tensor has only one dimension {x.shape}")  # mod.rs:363-365
        if x.shape[-1] != self.k:
            raise ValueError(f"input tensor {x.shape} incompatible with {(self.n, self.k)}")  # mod.rs:368-370
        m = int(np.prod(x.shape[:-1]))
        if out is not None and (out.dtype != np.float32 or not out.flags.c_contiguous or out.shape != x.shape[:-1] + (self.n,)):
            raise ValueError(f"out must be a contiguous float32 array of shape {x.shape[:-1] + (self.n,)}")
        y = out if out is not None else np.empty(x.shape[:-1] + (self.n,), np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, np.float32)
        if b is not None and b.shape != (self.n,):
            raise ValueError(f"bias shape {b.shape} does not match n={self.n}")
        with torch.cuda.device(self.device):
            check(_lib.lib().xnq_linear_forward_host(self._h, ctypes.c_void_p(x.ctypes.data), m,
                                                     ctypes.c_void_p(b.ctypes.data) if b is not None else None,
                                                     ctypes.c_void_p(y.ctypes.data), _stream_ptr(self.device)))
        return y


class QCudaLinear:
    """A linear layer with GGUF-quantized weights on the device (``Q8Linear``, q8.rs:160-185)."""

    def __init__(self, weight: QCudaTensor, bias: Optional[torch.Tensor] = None):
        if bias is not None and tuple(bias.shape) != (weight.n,):
            raise ValueError(f"bias shape {tuple(bias.shape)} does not match out_features {weight.n}")
        self.weight, self.bias = weight, bias

    @classmethod
    def new(cls, weight: QCudaTensor, bias: Optional[torch.Tensor] = None) -> "QCudaLinear":
        return cls(weight, bias)

    @classmethod
    def from_linear(cls, weight: torch.Tensor, dtype: GgmlDType, bias: Optional[torch.Tensor] = None) -> "QCudaLinear":
        """``QLinear::from_linear`` (mod.rs:398-405): quantize a dense linear's ``[out, in]`` weight."""
        return cls(QCudaTensor.from_dense(weight, dtype), bias)

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        if xs.dim() < 2:
            raise ValueError(f"input tensor has only one dimension {tuple(xs.shape)}")  # mod.rs:363-365
        out = self.weight.matmul_t(xs)
        return out if self.bias is None else out + self.bias.to(out.dtype)  # broadcast_add, q8.rs:172-175

    __call__ = forward


def quantize_weight(weight: torch.Tensor, dtype: GgmlDType) -> torch.Tensor:
    """Canonical GGUF blocks of a dense ``[n, k]`` device tensor as a uint8 device tensor, bit-identical
    to the reference's host quantizers (``GgmlType::from_float``, k_quants.rs:235-270, 636-661, 1418-1473,
    1801-1871)."""
    dtype = GgmlDType(dtype)
    if weight.dim() != 2:
        raise ValueError(f"quantize_weight wants a 2-d tensor, got {tuple(weight.shape)}")
    n, k = weight.shape
    if k % dtype.block_size:
        raise ValueError(f"quantized tensor must have their last dim divisible by block size {tuple(weight.shape)} {dtype.block_size}")  # mod.rs:267-272
    init(weight.device)
    w = weight.to(torch.float32).contiguous()
    out = torch.empty(max(n * dtype.row_bytes(k), 16), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        check(_lib.lib().xnq_quantize_weight(int(dtype), ctypes.c_void_p(w.data_ptr()), n, k, ctypes.c_void_p(out.data_ptr()), _stream_ptr(weight.device)))
    return out[: n * dtype.row_bytes(k)]


def quantize_act(x: torch.Tensor, act_dtype: GgmlDType) -> torch.Tensor:
    """Canonical Q8_0 / Q8_1 / Q8_K activation blocks of ``x`` ``[m, k]`` as a uint8 device tensor."""
    act_dtype = GgmlDType(act_dtype)
    if x.dim() != 2 or x.stride(-1) != 1:
        raise ValueError("quantize_act wants a 2-d tensor with contiguous rows")
    m, k = x.shape
    init(x.device)
    nbytes = m * (k // act_dtype.block_size) * act_dtype.type_size if k % act_dtype.block_size == 0 else 0
    out = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.lib().xnq_quantize_act(int(act_dtype), ctypes.c_void_p(x.data_ptr()), int(_TORCH_TO_XNQ[x.dtype]), m, k,
                                          x.stride(0) if m > 1 else k, ctypes.c_void_p(out.data_ptr()), _stream_ptr(x.device)))
    return out[:nbytes]


class _BackendQ:
    """``BackendQ`` for the CUDA device with one GGML weight format (lib.rs:141-156)."""
    DTYPE: GgmlDType

    @classmethod
    def linear_from_qtensor(cls, qt: QTensor, in_features: int, out_features: int, device="cuda:0", shard_rank: int = 0,
                            shard_count: int = 1) -> QCudaLinear:
        """The ``linear_load`` branch that takes a file's blocks as they are (q8.rs:203-213): dtype and
        shape must match; weight only, no bias."""
        if qt.dtype() != cls.DTYPE:
            raise ValueError(f"cuda {cls.DTYPE.name}: expected a {cls.DTYPE.name} tensor, got {qt.dtype().name}")
        if tuple(qt.shape()) != (out_features, in_features):
            raise ValueError(f"cuda {cls.DTYPE.name}: weight is {list(qt.shape())}, expected [{out_features}, {in_features}]")
        return QCudaLinear(QCudaTensor.from_qtensor(qt, device, shard_rank, shard_count), None)


class Q40(_BackendQ):
    DTYPE = GgmlDType.Q4_0


class Q80(_BackendQ):
    DTYPE = GgmlDType.Q8_0


class Q4K(_BackendQ):
    DTYPE = GgmlDType.Q4K


class Q6K(_BackendQ):
    DTYPE = GgmlDType.Q6K


# the remaining weight formats the reference instantiates as BackendQ (mod.rs:444-455): held as the file's blocks, one plain kernel each
class Q41(_BackendQ):
    DTYPE = GgmlDType.Q4_1


class Q50(_BackendQ):
    DTYPE = GgmlDType.Q5_0


class Q51(_BackendQ):
    DTYPE = GgmlDType.Q5_1


class Q2K(_BackendQ):
    DTYPE = GgmlDType.Q2K


class Q3K(_BackendQ):
    DTYPE = GgmlDType.Q3K


class Q5K(_BackendQ):
    DTYPE = GgmlDType.Q5K


__all__ = ["QTensor", "QCudaTensor", "QCudaLinear", "Q40", "Q41", "Q50", "Q51", "Q80", "Q2K", "Q3K", "Q4K", "Q5K", "Q6K", "GgmlDType", "XnqError", "init",
           "quantize_act"]
