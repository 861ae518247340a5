"""The fused decode-step operators against plain torch f32 math."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(scope="module", autouse=True)
def _init():
    from xn_b200 import quantized
    quantized.init(DEV)


def test_add_rmsnorm():
    from xn_b200 import decoder_ops as ops
    torch.manual_seed(0)
    for rows, d in [(1, 4096), (16, 4096), (3, 512), (2, 14336)]:
        x = torch.randn(rows, d, device=DEV); delta = torch.randn(rows, d, device=DEV); w = torch.rand(d, device=DEV) + 0.5
        for dl in (None, delta):
            xin = x.clone(); out = torch.empty_like(x)
            ops.add_rmsnorm(xin, dl, w, 1e-5, out)
            xs = x + dl if dl is not None else x
            ref = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * w
            assert torch.equal(xin, xs)                      # the residual stream is updated in place, exactly
            torch.testing.assert_close(out, ref, rtol=2e-5, atol=2e-6)
        parts = torch.randn(rows, 3 * d, device=DEV)                 # three summands per row, side by side
        xin = x.clone(); out = torch.empty_like(x)
        ops.add_rmsnorm(xin, parts, w, 1e-5, out)
        xs = x + parts.view(rows, 3, d)[:, 0] + parts.view(rows, 3, d)[:, 1] + parts.view(rows, 3, d)[:, 2]
        torch.testing.assert_close(xin, xs, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(out, xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * w, rtol=2e-5, atol=2e-6)


def test_swiglu():
    from xn_b200 import decoder_ops as ops
    torch.manual_seed(1)
    for rows, f in [(1, 14336), (16, 1792), (5, 512)]:
        gu = torch.randn(rows, 2 * f, device=DEV) * 3
        out = torch.empty(rows, f, device=DEV)
        ops.swiglu(gu, out)
        torch.testing.assert_close(out, F.silu(gu[:, :f]) * gu[:, f:], rtol=1e-5, atol=1e-6)


def _rope_ref(x, cos, sin):
    x1, x2 = x[..., :64], x[..., 64:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


@pytest.mark.parametrize("B,H,KV", [(1, 32, 8), (16, 4, 1), (2, 8, 8)])
def test_rope_store_and_attention(B, H, KV):
    from xn_b200 import decoder_ops as ops
    torch.manual_seed(2)
    hd, max_seq = 128, 96
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=DEV, dtype=torch.float32) / hd))
    ang = torch.arange(max_seq, device=DEV, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc = torch.zeros(B, KV, max_seq, hd, device=DEV, dtype=torch.bfloat16); vc = torch.zeros_like(kc)
    kr = torch.zeros(B, KV, max_seq, hd, device=DEV); vr = torch.zeros_like(kr)
    for pos_i in [0, 1, 2, 37]:
        pos = torch.tensor([pos_i], device=DEV, dtype=torch.int64)
        qkv = torch.randn(B, (H + 2 * KV) * hd, device=DEV)
        q_out = torch.empty(B, H, hd, device=DEV)
        ops.rope_kv_store(qkv, cos, sin, pos, q_out, kc, vc, H, KV)
        q, k, v = qkv.split([H * hd, KV * hd, KV * hd], -1)
        q_ref = _rope_ref(q.view(B, H, hd), cos[pos_i], sin[pos_i])
        kr[:, :, pos_i] = _rope_ref(k.view(B, KV, hd), cos[pos_i], sin[pos_i]); vr[:, :, pos_i] = v.view(B, KV, hd)
        torch.testing.assert_close(q_out, q_ref, rtol=1e-5, atol=1e-6)
        assert torch.equal(kc[:, :, pos_i], kr[:, :, pos_i].to(torch.bfloat16)) and torch.equal(vc[:, :, pos_i], vr[:, :, pos_i].to(torch.bfloat16))
    # fill the rest of the cache and attend from several positions
    kc.copy_(torch.randn_like(kr).to(torch.bfloat16)); vc.copy_(torch.randn_like(vr).to(torch.bfloat16))
    for pos_i in [0, 5, 63, 95]:
        pos = torch.tensor([pos_i], device=DEV, dtype=torch.int64)
        q = torch.randn(B, H, hd, device=DEV)
        out = torch.empty_like(q)
        ops.attn_decode(q, kc, vc, pos, out, H, KV)
        kk = kc[:, :, : pos_i + 1].float().repeat_interleave(H // KV, 1); vv = vc[:, :, : pos_i + 1].float().repeat_interleave(H // KV, 1)
        w = torch.softmax(torch.einsum("bhd,bhsd->bhs", q, kk) / math.sqrt(hd), -1)
        torch.testing.assert_close(out, torch.einsum("bhs,bhsd->bhd", w, vv), rtol=2e-4, atol=2e-5)
