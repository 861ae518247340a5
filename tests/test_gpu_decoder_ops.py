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


def test_embedding_rows_and_greedy_choice():
    from xn_b200 import decoder_ops as ops
    torch.manual_seed(3)
    table = (torch.randn(1000, 512, device=DEV) * 0.02).to(torch.bfloat16)
    for rows in (1, 16):
        tokens = torch.randint(0, 1000, (rows,), device=DEV)
        out = torch.full((rows, 512), float("nan"), device=DEV)
        ops.embed_rows(table, tokens, out)
        assert torch.equal(out, table.index_select(0, tokens).float())
    for rows, n in [(1, 32000), (16, 32000), (3, 7), (2, 128256)]:
        logits = torch.randn(rows, n, device=DEV)
        logits[0, n // 3] = logits[0, n - 1] = 9.0          # equal maxima: the first one wins
        if rows > 1:
            logits[1, :] = -1.5                               # a constant row: index 0
        tokens = torch.full((rows,), -7, device=DEV, dtype=torch.int64)
        pos = torch.tensor([41], device=DEV, dtype=torch.int64)
        ops.argmax_advance(logits, tokens, pos)
        assert torch.equal(tokens, logits.argmax(-1)), (rows, n)
        assert int(pos.item()) == 42
        ops.argmax_advance(logits, tokens, None)
        assert int(pos.item()) == 42


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


@pytest.mark.parametrize("B,H,KV", [(1, 32, 8), (3, 8, 2), (2, 4, 4)])
def test_rope_inside_the_attention_kernel_is_bit_identical(B, H, KV):
    """xnq_rope_attn_decode == xnq_rope_kv_store followed by xnq_attn_decode: outputs and both caches, over several steps."""
    from xn_b200 import decoder_ops as ops
    torch.manual_seed(9)
    hd, max_seq = 128, 160
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=DEV, dtype=torch.float32) / hd))
    ang = torch.arange(max_seq, device=DEV, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc = torch.randn(B, KV, max_seq, hd, device=DEV).to(torch.bfloat16); vc = torch.randn(B, KV, max_seq, hd, device=DEV).to(torch.bfloat16)
    kc2, vc2 = kc.clone(), vc.clone()
    for pos_i in [0, 1, 31, 32, 33, 95, 96, 150, 159]:   # first position, run boundaries, the last one
        pos = torch.tensor([pos_i], device=DEV, dtype=torch.int64)
        qkv = torch.randn(B, (H + 2 * KV) * hd, device=DEV)
        q = torch.empty(B, H, hd, device=DEV); want = torch.empty(B, H, hd, device=DEV); got = torch.full_like(want, float("nan"))
        ops.rope_kv_store(qkv, cos, sin, pos, q, kc, vc, H, KV)
        ops.attn_decode(q, kc, vc, pos, want, H, KV)
        ops.rope_attn_decode(qkv, cos, sin, pos, kc2, vc2, got, H, KV)
        assert torch.equal(got, want), (pos_i, float((got - want).abs().max()))
        assert torch.equal(kc2, kc) and torch.equal(vc2, vc), pos_i


def test_attention_workspace_reuse_and_position_range():
    """One workspace serves calls of different (batch, heads): the arrival counters sit at offsets that depend on the
    (sequence, head) index alone. A position outside the cache is reported through the status word, never NaN."""
    import ctypes
    from xn_b200 import decoder_ops as ops, _lib
    L = _lib.lib()
    torch.manual_seed(5)
    hd, max_seq = 128, 64

    def run(B, H, KV, pos_i, ws):
        kc = torch.randn(B, KV, max_seq, hd, device=DEV).to(torch.bfloat16); vc = torch.randn(B, KV, max_seq, hd, device=DEV).to(torch.bfloat16)
        q = torch.randn(B, H, hd, device=DEV); out = torch.full_like(q, float("nan"))
        pos = torch.tensor([pos_i], device=DEV, dtype=torch.int64)
        _lib.check(L.xnq_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), out.data_ptr(), B, H, KV, hd, max_seq, ws.data_ptr(), ws.numel(),
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        last = min(max(pos_i, 0), max_seq - 1)
        kk = kc[:, :, : last + 1].float().repeat_interleave(H // KV, 1); vv = vc[:, :, : last + 1].float().repeat_interleave(H // KV, 1)
        w = torch.softmax(torch.einsum("bhd,bhsd->bhs", q, kk) / math.sqrt(hd), -1)
        return out, torch.einsum("bhs,bhsd->bhd", w, vv)

    ws = torch.zeros(int(L.xnq_attn_decode_workspace_bytes(4, 8)), dtype=torch.uint8, device=DEV)
    for B, H, KV in [(4, 8, 2), (1, 32, 8), (2, 4, 4), (4, 8, 2), (1, 2, 1)]:   # every shape splits the sequence differently
        out, ref = run(B, H, KV, 40, ws)
        torch.testing.assert_close(out, ref, rtol=2e-4, atol=2e-5)
    st = ctypes.c_uint()
    _lib.check(L.xnq_device_status(ctypes.byref(st)))
    assert st.value >> 24 == 0
    out, ref = run(2, 4, 2, max_seq + 5, ws)           # past the cache: clamped and flagged
    torch.testing.assert_close(out, ref, rtol=2e-4, atol=2e-5)
    out, _ = run(2, 4, 2, -1, ws)                      # nothing to attend to: zeros and flagged
    assert torch.equal(out, torch.zeros_like(out))
    _lib.check(L.xnq_device_status(ctypes.byref(st)))
    assert (st.value >> 24) & 2
    # the store kernel writes nothing for a position outside the cache
    H, KV = 4, 2
    qkv = torch.randn(1, (H + 2 * KV) * hd, device=DEV)
    cos = torch.ones(max_seq, hd // 2, device=DEV); sin = torch.zeros(max_seq, hd // 2, device=DEV)
    kc = torch.zeros(1, KV, max_seq, hd, device=DEV, dtype=torch.bfloat16); vc = torch.zeros_like(kc); q_out = torch.zeros(1, H, hd, device=DEV)
    ops.rope_kv_store(qkv, cos, sin, torch.tensor([max_seq], device=DEV, dtype=torch.int64), q_out, kc, vc, H, KV)
    assert not kc.any() and not vc.any() and not q_out.any()
    _lib.check(L.xnq_device_status(ctypes.byref(st)))
    assert (st.value >> 24) & 1
    _lib.check(L.xnq_init(0))                          # clears the sticky bits for the tests that follow
    _lib.check(L.xnq_device_status(ctypes.byref(st)))
    assert st.value == 0


@pytest.mark.parametrize("m", [2, 7, 16, 17, 32, 33, 64])
def test_operand_images_give_the_bits_of_the_other_input_forms(m):
    """add_rmsnorm / swiglu writing the integer tensor-core kernel's operand layout (XNQ_ACT_OPERAND): the matmul on it, one
    kernel, must equal bit for bit the matmul on float rows; an image may feed several matmuls in turn (the ticket words of
    split tiles are put back by the kernel that used them)."""
    from xn_b200 import decoder_ops as ops, quantized as Q, synth
    from xn_b200.dtypes import GgmlDType as D
    Q.init(DEV)
    torch.manual_seed(31 + m)
    for n, k in [(300, 256), (6144, 4096), (520, 11008)]:
        w = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(D.Q4K, n, k, seed=90), (n, k), D.Q4K), DEV)
        w2 = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(D.Q4K, 130, k, seed=91), (130, k), D.Q4K), DEV)
        x = torch.randn(m, k, device=DEV) * 2; g = torch.rand(k, device=DEV) + 0.5
        x[0, :40] = 0.0
        xn = torch.empty(m, k, device=DEV)
        img = ops.OperandImage(m, k, DEV)
        ops.add_rmsnorm(x.clone(), None, g, 1e-5, xn, img)
        want = w.matmul_t(xn)
        for rep in range(2):   # the second use finds the tickets as the first one left them
            got = w.matmul_t(img)
            assert torch.equal(got, want), ("norm", m, n, k, rep, float((got - want).abs().max()))
        assert torch.equal(w2.matmul_t(img), w2.matmul_t(xn)), ("norm, second weight", m, k)
        gu = torch.randn(m, 2 * k, device=DEV) * 2
        h = torch.empty(m, k, device=DEV)
        ops.swiglu(gu, h, img)   # the same image object, rewritten
        want = w.matmul_t(h)
        got = w.matmul_t(img)
        assert torch.equal(got, want), ("swiglu", m, n, k, float((got - want).abs().max()))


def test_activation_images_equal_the_in_call_quantizer():
    """An image written by the stand-alone quantizer, by add_rmsnorm or by swiglu holds the bytes the matmul's own
    quantizer would produce from the same f32 rows, so matmul results through an image are bit-identical."""
    from xn_b200 import decoder_ops as ops, quantized as Q, synth
    from xn_b200.dtypes import GgmlDType as D
    torch.manual_seed(3)
    for dt, n, k in [(D.Q4K, 320, 4096), (D.Q6K, 96, 1024), (D.Q8_0, 200, 4096), (D.Q4_0, 64, 512), (D.Q4K, 128, 14336)]:
        w = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(dt, n, k, seed=40), (n, k), dt), DEV)
        for m in (1, 3, 16):
            x = torch.randn(m, k, device=DEV)
            want = w.matmul_t(x)
            img = ops.quantize_act_image(x, ops.ActImage.for_weight(dt, m, k, DEV))
            assert torch.equal(w.matmul_t(img), want), (dt.name, k, m, "quantize_act_image")
            # add_rmsnorm: the image equals the quantization of its own f32 output
            res = torch.randn(m, k, device=DEV); dl = torch.randn(m, k, device=DEV); g = torch.rand(k, device=DEV) + 0.5
            out = torch.empty(m, k, device=DEV); img2 = ops.ActImage.for_weight(dt, m, k, DEV)
            ops.add_rmsnorm(res.clone(), dl, g, 1e-5, out, img2)
            assert torch.equal(w.matmul_t(img2), w.matmul_t(out)), (dt.name, k, m, "add_rmsnorm")
            only = ops.ActImage.for_weight(dt, m, k, DEV)
            ops.add_rmsnorm(res.clone(), dl, g, 1e-5, None, only)      # image without the f32 rows
            assert torch.equal(w.matmul_t(only), w.matmul_t(img2))
            if k % 256 == 0:
                gu = torch.randn(m, 2 * k, device=DEV) * 2
                h = torch.empty(m, k, device=DEV); img3 = ops.ActImage.for_weight(dt, m, k, DEV)
                ops.swiglu(gu, h, img3)
                assert torch.equal(w.matmul_t(img3), w.matmul_t(h)), (dt.name, k, m, "swiglu")
    with pytest.raises(ValueError):
        w.matmul_t(ops.ActImage.for_weight(D.Q8_0, 1, 14336, DEV))   # a Q8_0 image does not fit a Q4_K weight
