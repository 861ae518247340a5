"""Seeded synthetic GGUF blocks and activations with the benchmark configurations' distributions.

No GGUF file or model weight is available offline, so every tensor the tests and the benchmark
use is generated here: block scales are ``f16(|N(0,1)| * dscale)``, codes are uniform over the
format's code range, activations are N(0,1) f32.  The byte layouts are the canonical GGUF ones
(xn-core/src/quantized/k_quants.rs:92-196), which is what ``QTensor::data()`` yields and what
the device upload takes.

Rows are generated in groups of ``ROW_GROUP`` with an RNG stream keyed by
``(seed, tensor_id, group index)``, so a rank that holds rows ``[r0, r1)`` of an N-sharded
weight generates exactly the bytes the unsharded tensor has there.
"""
from __future__ import annotations

import numpy as np

from .dtypes import GgmlDType

ROW_GROUP = 32


def _rng(seed: int, tensor_id: int, group: int) -> np.random.Generator:
    return np.random.default_rng([int(seed), int(tensor_id), int(group)])


def _f16_bytes(x: np.ndarray) -> np.ndarray:
    """f32 -> IEEE binary16 (round-to-nearest-even) as little-endian byte pairs."""
    return x.astype(np.float16).view(np.uint8).reshape(*x.shape, 2)


def pack_q4_0(d: np.ndarray, codes: np.ndarray) -> np.ndarray:
    """d: [R, B] f32, codes: [R, B, 32] in 0..15 -> [R, B, 18] bytes.

    Element j sits in the low nibble of qs[j], element j+16 in the high nibble
    (k_quants.rs:213-233)."""
    r, b = d.shape
    out = np.empty((r, b, 18), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = codes[..., :16] | (codes[..., 16:] << 4)
    return out


def pack_q8_0(d: np.ndarray, codes: np.ndarray) -> np.ndarray:
    """d: [R, B] f32, codes: [R, B, 32] int8 -> [R, B, 34] bytes (k_quants.rs:128-134)."""
    r, b = d.shape
    out = np.empty((r, b, 34), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = codes.astype(np.int8).view(np.uint8)
    return out


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Eight 6-bit scales and eight 6-bit mins -> the 12-byte field of a Q4_K block.

    The inverse of ``get_scale_min_k4`` (xn-core/src/quantized/utils.rs:53-63; the packing
    the reference's own quantizer uses is k_quants.rs:1434-1445)."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.empty(sc.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return out


def pack_q4_k(d, dmin, sc, mn, codes) -> np.ndarray:
    """d, dmin: [R, B]; sc, mn: [R, B, 8] in 0..63; codes: [R, B, 256] in 0..15 -> [R, B, 144].

    Each 32-byte chunk c of qs holds sub-block 2c in the low nibbles and 2c+1 in the high ones
    (k_quants.rs:1475-1503)."""
    r, b = d.shape
    out = np.empty((r, b, 144), np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(dmin)
    out[..., 4:16] = pack_scales_k4(sc, mn)
    c = codes.reshape(r, b, 4, 2, 32).astype(np.uint8)
    out[..., 16:] = (c[:, :, :, 0, :] | (c[:, :, :, 1, :] << 4)).reshape(r, b, 128)
    return out


def pack_q6_k(d, scales, codes) -> np.ndarray:
    """d: [R, B]; scales: [R, B, 16] int8; codes: [R, B, 256] in 0..63 -> [R, B, 210].

    Per 128-element half h and l in 0..32, the four elements l, l+32, l+64, l+96 take their low
    nibbles from ql[l] / ql[l+32] (low, low, high, high) and their top two bits from the four
    bit pairs of qh[l] (k_quants.rs:1874-1904).  d is the LAST field of the block."""
    r, b = d.shape
    c = codes.reshape(r, b, 2, 4, 32).astype(np.uint8)  # [half, group, l]
    lo, hi = c & 0xF, c >> 4
    ql = np.empty((r, b, 2, 64), np.uint8)
    ql[..., 0:32] = lo[:, :, :, 0, :] | (lo[:, :, :, 2, :] << 4)
    ql[..., 32:64] = lo[:, :, :, 1, :] | (lo[:, :, :, 3, :] << 4)
    qh = hi[:, :, :, 0, :] | (hi[:, :, :, 1, :] << 2) | (hi[:, :, :, 2, :] << 4) | (hi[:, :, :, 3, :] << 6)
    out = np.empty((r, b, 210), np.uint8)
    out[..., 0:128] = ql.reshape(r, b, 128)
    out[..., 128:192] = qh.reshape(r, b, 64)
    out[..., 192:208] = scales.astype(np.int8).view(np.uint8)
    out[..., 208:210] = _f16_bytes(d)
    return out


# default |N(0,1)| multipliers of the block scales, per the benchmark configurations
DEFAULT_DSCALE = {
    GgmlDType.Q4_0: 0.02,
    GgmlDType.Q8_0: 0.01,
    GgmlDType.Q4K: 0.01,
    GgmlDType.Q6K: 0.005,
    GgmlDType.Q4_1: 0.02,
    GgmlDType.Q5_0: 0.01,
    GgmlDType.Q5_1: 0.01,
    GgmlDType.Q2K: 0.01,
    GgmlDType.Q3K: 0.01,
    GgmlDType.Q5K: 0.005,
}


def _gen_group(dtype: GgmlDType, rows: int, k: int, dscale: float, g: np.random.Generator) -> np.ndarray:
    nb = k // dtype.block_size
    if dtype == GgmlDType.Q4_0:
        d = np.abs(g.standard_normal((rows, nb), np.float32)) * np.float32(dscale)
        return pack_q4_0(d, g.integers(0, 16, (rows, nb, 32), np.uint8))
    if dtype == GgmlDType.Q8_0:
        d = np.abs(g.standard_normal((rows, nb), np.float32)) * np.float32(dscale)
        return pack_q8_0(d, g.integers(-127, 128, (rows, nb, 32), np.int8))
    if dtype == GgmlDType.Q4K:
        d = np.abs(g.standard_normal((rows, nb), np.float32)) * np.float32(dscale)
        dmin = np.abs(g.standard_normal((rows, nb), np.float32)) * np.float32(dscale)
        sc = g.integers(0, 64, (rows, nb, 8), np.uint8)
        mn = g.integers(0, 64, (rows, nb, 8), np.uint8)
        return pack_q4_k(d, dmin, sc, mn, g.integers(0, 16, (rows, nb, 256), np.uint8))
    if dtype == GgmlDType.Q6K:
        d = np.abs(g.standard_normal((rows, nb), np.float32)) * np.float32(dscale)
        sc = g.integers(-64, 64, (rows, nb, 16), np.int8)
        return pack_q6_k(d, sc, g.integers(0, 64, (rows, nb, 256), np.uint8))
    # The formats beyond the four of the benchmark configurations: random valid blocks laid out as the reference's
    # #[repr(C)] structs (k_quants.rs:100-186): f16 scales from |N(0,1)| * dscale, every code / scale / mask bit uniform.
    f16s = lambda: _f16_bytes(np.abs(g.standard_normal((rows, nb), np.float32)) * np.float32(dscale))   # noqa: E731
    rnd = lambda n: g.integers(0, 256, (rows, nb, n), np.uint8)                                          # noqa: E731
    out = np.empty((rows, nb, dtype.type_size), np.uint8)
    if dtype == GgmlDType.Q4_1:     # {f16 d; f16 m; u8 qs[16]}
        out[..., 0:2], out[..., 2:4], out[..., 4:20] = f16s(), _f16_bytes(g.standard_normal((rows, nb), np.float32) * np.float32(dscale * 4)), rnd(16)
    elif dtype == GgmlDType.Q5_0:   # {f16 d; u8 qh[4]; u8 qs[16]}
        out[..., 0:2], out[..., 2:6], out[..., 6:22] = f16s(), rnd(4), rnd(16)
    elif dtype == GgmlDType.Q5_1:   # {f16 d; f16 m; u8 qh[4]; u8 qs[16]}
        out[..., 0:2], out[..., 2:4] = f16s(), _f16_bytes(g.standard_normal((rows, nb), np.float32) * np.float32(dscale * 8))
        out[..., 4:8], out[..., 8:24] = rnd(4), rnd(16)
    elif dtype == GgmlDType.Q2K:    # {u8 scales[16]; u8 qs[64]; f16 d; f16 dmin}
        out[..., 0:16], out[..., 16:80], out[..., 80:82], out[..., 82:84] = rnd(16), rnd(64), f16s(), f16s()
    elif dtype == GgmlDType.Q3K:    # {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d}
        out[..., 0:32], out[..., 32:96], out[..., 96:108], out[..., 108:110] = rnd(32), rnd(64), rnd(12), f16s()
    elif dtype == GgmlDType.Q5K:    # {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}
        out[..., 0:2], out[..., 2:4], out[..., 4:16], out[..., 16:48], out[..., 48:176] = f16s(), f16s(), rnd(12), rnd(32), rnd(128)
    else:
        raise ValueError(f"no synthetic generator for {dtype}")
    return out


def make_weight(dtype: GgmlDType, n: int, k: int, seed: int = 0, tensor_id: int = 0,
                dscale: float | None = None, rows: tuple[int, int] | None = None) -> np.ndarray:
    """Canonical GGUF bytes of a synthetic ``[n, k]`` weight (or of its rows ``[r0, r1)``).

    Returns a flat uint8 array of ``(r1 - r0) * (k / block) * type_size`` bytes."""
    dtype = GgmlDType(dtype)
    if k % dtype.block_size:
        raise ValueError(f"k={k} is not a multiple of the {dtype.block_size}-element block")
    r0, r1 = (0, n) if rows is None else rows
    if not (0 <= r0 <= r1 <= n):
        raise ValueError(f"rows {rows} outside [0, {n}]")
    dscale = DEFAULT_DSCALE[dtype] if dscale is None else dscale
    row_bytes = dtype.row_bytes(k)
    out = np.empty((r1 - r0, row_bytes), np.uint8)
    for grp in range(r0 // ROW_GROUP, (max(r1, 1) - 1) // ROW_GROUP + 1 if r1 > r0 else 0):
        g0, g1 = grp * ROW_GROUP, min((grp + 1) * ROW_GROUP, n)
        blk = _gen_group(dtype, g1 - g0, k, dscale, _rng(seed, tensor_id, grp)).reshape(g1 - g0, row_bytes)
        lo, hi = max(g0, r0), min(g1, r1)
        out[lo - r0:hi - r0] = blk[lo - g0:hi - g0]
    return out.reshape(-1)


def make_activation(m: int, k: int, seed: int = 0, tensor_id: int = 1000) -> np.ndarray:
    """f32 ``[m, k]`` activations drawn from N(0,1)."""
    return _rng(seed, tensor_id, 0).standard_normal((m, k), np.float32)
