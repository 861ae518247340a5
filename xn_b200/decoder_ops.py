"""Torch-tensor wrappers of the fused decode-step operators (``xnq_add_rmsnorm``, ``xnq_swiglu``,
``xnq_rope_kv_store``, ``xnq_attn_decode``): the pieces of the reference's Llama block between its
linears (xn-core/src/models/llama.rs:145-216, 258-265, 300-320)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .dtypes import GgmlDType
from .quantized import _stream_ptr


class ActImage:
    """Activations quantized ahead of the matmul: ``m`` rows of ``k`` values as Q8_0 or Q8_K codes, block scales
    and 16-element sums in the planar layout the decode kernels read (``xnq_act_image_bytes``). Written by
    ``add_rmsnorm`` / ``swiglu`` / ``quantize_act_image``, read by ``QCudaTensor.matmul_t``."""

    def __init__(self, act_dtype: GgmlDType, m: int, k: int, device: torch.device):
        self.act_dtype, self.m, self.k, self.device = GgmlDType(act_dtype), m, k, device
        nbytes = int(_lib.lib().xnq_act_image_bytes(int(self.act_dtype), m, k))
        if nbytes == 0:
            raise ValueError(f"no activation image for {self.act_dtype.name} [{m}, {k}]")
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    @classmethod
    def for_weight(cls, weight_dtype: GgmlDType, m: int, k: int, device: torch.device) -> "ActImage":
        return cls(GgmlDType(weight_dtype).vec_dot_type, m, k, device)

    def data_ptr(self) -> int:
        return self.buf.data_ptr()


class OperandImage:
    """Up to 64 activation rows quantized to Q8_K in the layout the integer tensor-core kernel reads (``XNQ_ACT_OPERAND``), with
    the ticket words of its split tiles: written by ``add_rmsnorm`` / ``swiglu``, read by ``QCudaTensor.matmul_t`` on Q4_K weights,
    which then is one kernel. Zeroed at creation (the padded rows and the tickets are never written by a producer); belongs to one
    ``(m, k)``; one matmul at a time may read it."""
    operand = True

    def __init__(self, m: int, k: int, device: torch.device):
        self.act_dtype, self.m, self.k, self.device = GgmlDType.Q8K, m, k, device
        nbytes = int(_lib.lib().xnq_act_operand_bytes(m, k))
        if nbytes == 0:
            raise ValueError(f"no operand image for [{m}, {k}] (1..64 rows, k a multiple of 256)")
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)

    def data_ptr(self) -> int:
        return self.buf.data_ptr()


def quantize_act_image(x: torch.Tensor, image: ActImage) -> ActImage:
    """Quantize ``x [m, k]`` (f32 / f16 / bf16, contiguous rows) into ``image``."""
    from .quantized import _TORCH_TO_XNQ
    m, k = x.shape
    if (m, k) != (image.m, image.k) or x.stride(-1) != 1:
        raise ValueError(f"image is [{image.m}, {image.k}], x is {tuple(x.shape)}")
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().xnq_quantize_act_image(int(image.act_dtype), _p(x), int(_TORCH_TO_XNQ[x.dtype]), m, k, x.stride(0) if m > 1 else k,
                                                     ctypes.c_void_p(image.data_ptr()), _stream_ptr(x.device)))
    return image


def _img(image: Optional[ActImage], rows: int, k: int):
    if image is None:
        return None, 0
    if (image.m, image.k) != (rows, k):
        raise ValueError(f"image is [{image.m}, {image.k}], rows are [{rows}, {k}]")
    return ctypes.c_void_p(image.data_ptr()), (_lib.XNQ_ACT_OPERAND if getattr(image, "operand", False) else int(image.act_dtype))


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _f32c(*ts):
    for t in ts:
        if t is not None and (t.dtype is not torch.float32 or not t.is_contiguous()):
            raise ValueError("expected contiguous float32 tensors")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
                image: Optional[ActImage] = None) -> Optional[torch.Tensor]:
    """In place ``x += delta`` (skipped when ``delta`` is None), then ``out = rmsnorm(x) * weight``; ``x`` is ``[rows, d]``.
    ``delta`` may be ``[rows, parts * d]``: its ``parts`` summands per row are all added. ``image`` also receives the
    quantized form of the normalized rows (the bytes quantizing ``out`` would give)."""
    _f32c(x, delta, weight, out)
    rows, d = x.shape
    parts = 1 if delta is None else delta.numel() // (rows * d)
    ip, idt = _img(image, rows, d)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().xnq_add_rmsnorm(_p(x), _p(delta), parts, _p(weight), eps, _p(out), ip, idt, rows, d, _stream_ptr(x.device)))
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, image: Optional[ActImage] = None) -> Optional[torch.Tensor]:
    """``out[rows, f] = silu(gate_up[:, :f]) * gate_up[:, f:]``, optionally with its quantized image."""
    _f32c(gate_up, out)
    rows, f2 = gate_up.shape
    ip, idt = _img(image, rows, f2 // 2)
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.lib().xnq_swiglu(_p(gate_up), _p(out), ip, idt, rows, f2 // 2, _stream_ptr(gate_up.device)))
    return out


def embed_rows(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[r, :] = table[tokens[r], :]`` widened to f32 (bf16 table ``[vocab, d]``, int64 tokens): the embedding lookup of a
    decode step as one plain launch (xnq_embed_rows)."""
    if table.dtype is not torch.bfloat16 or tokens.dtype is not torch.int64 or out.dtype is not torch.float32:
        raise ValueError("embed_rows: bf16 table, int64 tokens, f32 output")
    if not (table.is_contiguous() and tokens.is_contiguous() and out.is_contiguous()):
        raise ValueError("embed_rows: contiguous tensors")
    rows, d = tokens.numel(), table.shape[1]
    if out.numel() != rows * d:
        raise ValueError("embed_rows: output shape")
    with torch.cuda.device(table.device):
        _lib.check(_lib.lib().xnq_embed_rows(_p(table), _p(tokens), _p(out), rows, d, table.shape[0], _stream_ptr(table.device)))
    return out


def argmax_advance(logits: torch.Tensor, tokens: torch.Tensor, pos: Optional[torch.Tensor]) -> None:
    """``tokens[r] = argmax(logits[r])`` (first of equal maxima), then ``pos += 1``: the greedy choice and the position advance of
    a decode step in one launch (xnq_argmax_advance)."""
    if logits.dtype is not torch.float32 or not logits.is_contiguous() or tokens.dtype is not torch.int64 or (pos is not None and pos.dtype is not torch.int64):
        raise ValueError("argmax_advance: f32 contiguous logits, int64 tokens and position")
    rows, n = logits.shape
    if tokens.numel() != rows:
        raise ValueError("argmax_advance: one token per row")
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().xnq_argmax_advance(_p(logits), rows, n, _p(tokens), _p(pos), _stream_ptr(logits.device)))


def rope_kv_store(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, heads: int, kv_heads: int) -> None:
    """One token per sequence: rotate q and k at ``pos`` (int64 device scalar), write q to ``q_out [B, heads, hd]``
    and k, v (bf16) into the caches ``[B, kv_heads, max_seq, hd]`` at that position."""
    _f32c(qkv, cos, sin, q_out)
    B, _, max_seq, hd = k_cache.shape
    if k_cache.dtype is not torch.bfloat16 or not k_cache.is_contiguous() or not v_cache.is_contiguous() or pos.dtype is not torch.int64:
        raise ValueError("caches must be contiguous bfloat16 and pos int64")
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.lib().xnq_rope_kv_store(_p(qkv), _p(cos), _p(sin), _p(pos), _p(q_out), _p(k_cache), _p(v_cache), B, heads, kv_heads, hd,
                                                max_seq, _stream_ptr(qkv.device)))


_attn_ws: dict[tuple[int, int], torch.Tensor] = {}   # (device, stream) -> workspace, grown on demand


def _attn_workspace(device: torch.device, B: int, heads: int) -> torch.Tensor:
    L = _lib.lib()
    key = (device.index or 0, int(_stream_ptr(device).value or 0))   # calls on different streams may overlap: one workspace each
    need = max(int(L.xnq_attn_decode_workspace_bytes(B, heads)), 16)
    ws = _attn_ws.get(key)
    if ws is None or ws.numel() < need:   # zeroed once; the kernel leaves its arrival counters at zero
        ws = _attn_ws[key] = torch.zeros(need, dtype=torch.uint8, device=device)
    return ws


def rope_attn_decode(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     out: torch.Tensor, heads: int, kv_heads: int) -> torch.Tensor:
    """:func:`rope_kv_store` and :func:`attn_decode` in one launch (same bits): rotates q and the new k inside the attention
    kernel, which also stores the new k and v into the caches. ``qkv`` is ``[B, (heads + 2 kv_heads) * hd]``."""
    _f32c(qkv, cos, sin, out)
    B, _, max_seq, hd = k_cache.shape
    if k_cache.dtype is not torch.bfloat16 or not k_cache.is_contiguous() or not v_cache.is_contiguous() or pos.dtype is not torch.int64:
        raise ValueError("rope_attn_decode: caches must be contiguous bf16 [B, kv_heads, max_seq, hd] and pos an int64 device scalar")
    ws = _attn_workspace(qkv.device, B, heads)
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.lib().xnq_rope_attn_decode(_p(qkv), _p(cos), _p(sin), _p(pos), _p(k_cache), _p(v_cache), _p(out), B, heads, kv_heads, hd, max_seq,
                                                    _p(ws), ws.numel(), _stream_ptr(qkv.device)))
    return out


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int) -> torch.Tensor:
    """Single-query attention over cache positions ``0..pos``; ``q`` and ``out`` are ``[B, heads, hd]``."""
    _f32c(q, out)
    B, _, max_seq, hd = k_cache.shape
    L = _lib.lib()
    ws = _attn_workspace(q.device, B, heads)
    with torch.cuda.device(q.device):
        _lib.check(L.xnq_attn_decode(_p(q), _p(k_cache), _p(v_cache), _p(pos), _p(out), B, heads, kv_heads, hd, max_seq, _p(ws), ws.numel(),
                                     _stream_ptr(q.device)))
    return out
