"""A second, independent restatement (numpy) of the block unpackers and the two activation
quantizers, written from the reference text and used only to cross-check the C oracle.

to_float: xn-core/src/quantized/k_quants.rs:213-233 (Q4_0), 618-634 (Q8_0), 1475-1503 (Q4_K),
1874-1904 (Q6_K).  from_float: 636-661 (Q8_0), 1942-1979 (Q8_K)."""
import numpy as np


def _f16(b):  # [..., 2] bytes -> f32
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)[..., 0]


def to_float_q4_0(raw, nelem):
    blk = raw.reshape(-1, 18)
    d = _f16(blk[:, 0:2])[:, None]
    qs = blk[:, 2:]
    lo = (qs & 0xF).astype(np.int32) - 8
    hi = (qs >> 4).astype(np.int32) - 8
    return (np.concatenate([lo, hi], 1).astype(np.float32) * d).reshape(nelem)


def to_float_q8_0(raw, nelem):
    blk = raw.reshape(-1, 34)
    d = _f16(blk[:, 0:2])[:, None]
    return (blk[:, 2:].view(np.int8).astype(np.float32) * d).reshape(nelem)


def scale_min_k4(scales):  # [B, 12] -> sc [B, 8], mn [B, 8]  (utils.rs:53-63)
    q = scales.astype(np.uint8)
    sc = np.empty(q.shape[:-1] + (8,), np.uint8)
    mn = np.empty_like(sc)
    for j in range(8):
        if j < 4:
            sc[..., j] = q[..., j] & 63
            mn[..., j] = q[..., j + 4] & 63
        else:
            sc[..., j] = (q[..., j + 4] & 0xF) | ((q[..., j - 4] >> 6) << 4)
            mn[..., j] = (q[..., j + 4] >> 4) | ((q[..., j] >> 6) << 4)
    return sc, mn


def to_float_q4k(raw, nelem):
    blk = raw.reshape(-1, 144)
    d = _f16(blk[:, 0:2])
    dmin = _f16(blk[:, 2:4])
    sc, mn = scale_min_k4(blk[:, 4:16])
    qs = blk[:, 16:].reshape(-1, 4, 32)
    out = np.empty((blk.shape[0], 8, 32), np.float32)
    for c in range(4):
        for half, codes in ((0, qs[:, c] & 0xF), (1, qs[:, c] >> 4)):
            j = 2 * c + half
            d1 = (d * sc[:, j].astype(np.float32))[:, None]
            m1 = (dmin * mn[:, j].astype(np.float32))[:, None]
            out[:, j] = d1 * codes.astype(np.float32) - m1
    return out.reshape(nelem)


def to_float_q6k(raw, nelem):
    blk = raw.reshape(-1, 210)
    ql = blk[:, 0:128].reshape(-1, 2, 64)
    qh = blk[:, 128:192].reshape(-1, 2, 32)
    sc = blk[:, 192:208].view(np.int8).reshape(-1, 2, 8).astype(np.float32)
    d = _f16(blk[:, 208:210])
    out = np.empty((blk.shape[0], 2, 4, 32), np.float32)
    l = np.arange(32)
    for h in range(2):
        a, b, hb = ql[:, h, :32], ql[:, h, 32:], qh[:, h]
        q = [
            ((a & 0xF) | ((hb & 3) << 4)).astype(np.int32) - 32,
            ((b & 0xF) | (((hb >> 2) & 3) << 4)).astype(np.int32) - 32,
            ((a >> 4) | (((hb >> 4) & 3) << 4)).astype(np.int32) - 32,
            ((b >> 4) | (((hb >> 6) & 3) << 4)).astype(np.int32) - 32,
        ]
        for g in range(4):
            s = sc[:, h][:, l // 16 + 2 * g]
            out[:, h, g] = (d[:, None] * s) * q[g].astype(np.float32)
    return out.reshape(nelem)


TO_FLOAT = {2: to_float_q4_0, 8: to_float_q8_0, 12: to_float_q4k, 14: to_float_q6k}


def _round_away(v):
    return np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5))).astype(np.float32)


def round_half_away(v):
    """f32::round. floor(v+0.5) is wrong when v+0.5 rounds up in f32, so go through trunc."""
    v = v.astype(np.float32)
    t = np.trunc(v)
    frac = np.abs(v - t)
    return np.where(frac >= np.float32(0.5), t + np.sign(v), t).astype(np.float32)


def from_float_q8_0(x):
    x = x.astype(np.float32).reshape(-1, 32)
    amax = np.abs(x).max(1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    q = np.clip(round_half_away(x * inv[:, None]), -128, 127).astype(np.int8)
    out = np.empty((x.shape[0], 34), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def from_float_q8k(x):
    x = x.astype(np.float32).reshape(-1, 256)
    idx = np.argmax(np.abs(x), 1)  # first index of the maximum, like the strict `<` scan
    mx = x[np.arange(x.shape[0]), idx]
    out = np.zeros((x.shape[0], 292), np.uint8)
    nz = mx != 0
    with np.errstate(divide="ignore", invalid="ignore"):
        iscale = (np.float32(-128.0) / mx).astype(np.float32)
        v = np.minimum(round_half_away(iscale[:, None] * x), np.float32(127.0))
        q = np.clip(v, -128, 127).astype(np.int8)
        d = (np.float32(1.0) / iscale).astype(np.float32)
    q[~nz] = 0
    d[~nz] = 0
    bs = q.reshape(-1, 16, 16).astype(np.int32).sum(2).astype(np.int16)
    out[:, 0:4] = d.view(np.uint8).reshape(-1, 4)
    out[:, 4:260] = q.view(np.uint8)
    out[:, 260:292] = bs.view(np.uint8).reshape(-1, 32)
    return out.reshape(-1)
