"""The decoder harness on a tiny configuration: quantized path vs dense math on the dequantized weights,
KV-cache consistency, graph replay, and tensor parallelism over two GPUs when present."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a - b).norm() / b.norm())


def test_tiny_decoder_matches_dense_math_and_its_own_cache():
    from xn_b200.llama import LlamaConfig, QLlama, dense_reference_logits
    dev = torch.device("cuda", 0)
    m = QLlama(LlamaConfig.tiny(), dev, batch=2, max_seq=64, max_prefill_rows=64)
    g = torch.Generator(device="cpu"); g.manual_seed(5)
    prompt = torch.randint(0, m.cfg.vocab, (2, 12), generator=g).to(dev)
    logits = m.prefill(prompt)
    ref = dense_reference_logits(m, prompt)
    assert logits.shape == (2, m.cfg.vocab)
    assert _rel(logits, ref) < 3e-2, _rel(logits, ref)      # Q8 activation blocks + bf16 attention vs f32 dense
    # one decode step through the cache == prefill of the extended prompt
    nxt = m.tokens.clone()
    m._decode_step()
    step_logits = m.last_logits.clone()
    m2 = QLlama(LlamaConfig.tiny(), dev, batch=2, max_seq=64, max_prefill_rows=64)
    full = m2.prefill(torch.cat([prompt, nxt[:, None]], dim=1))
    assert _rel(step_logits, full) < 2e-2, _rel(step_logits, full)


def test_graph_replay_generates_what_eager_decode_generates():
    from xn_b200.llama import LlamaConfig, QLlama
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu"); g.manual_seed(6)
    prompt = torch.randint(0, 512, (1, 9), generator=g).to(dev)
    a = QLlama(LlamaConfig.tiny(), dev, batch=1, max_seq=64, max_prefill_rows=64)
    a.prefill(prompt)
    eager = a.decode(10)
    b = QLlama(LlamaConfig.tiny(), dev, batch=1, max_seq=64, max_prefill_rows=64)
    b.prefill(prompt)
    b.capture_decode()
    replayed = b.decode(10)
    assert torch.equal(eager, replayed)
    assert int(b.pos.item()) == 19


def test_fused_decode_step_agrees_with_the_torch_op_decode_step():
    from xn_b200.llama import LlamaConfig, QLlama
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu"); g.manual_seed(8)
    prompt = torch.randint(0, 512, (3, 11), generator=g).to(dev)
    logits = []
    for fused in (True, False):
        m = QLlama(LlamaConfig.tiny(), dev, batch=3, max_seq=64, max_prefill_rows=64, fused_decode=fused)
        m.prefill(prompt)
        for _ in range(3):
            m._decode_step()
        logits.append(m.last_logits.clone())
    # torch's attention runs on bf16 q and rounds its output to bf16; the fused one keeps f32
    assert _rel(logits[0], logits[1]) < 3e-2, _rel(logits[0], logits[1])


def test_norm_in_the_matvec_prologue_is_bit_identical_to_the_separate_kernels():
    """One row: xnq_matvec_normed (residual add + RMSNorm + quantizer in the matvec's prologue) against
    xnq_add_rmsnorm with an image followed by the matmul, for every format; then a whole decoder with and without it."""
    from xn_b200 import decoder_ops as ops, quantized as Q, synth
    from xn_b200.dtypes import GgmlDType as D
    from xn_b200.llama import LlamaConfig, QLlama
    dev = torch.device("cuda", 0)
    Q.init(dev)
    torch.manual_seed(11)
    for dt, n, k, parts in [(D.Q4K, 6144, 4096, 1), (D.Q4K, 320, 1024, 0), (D.Q6K, 1000, 4096, 2), (D.Q8_0, 256, 2048, 1), (D.Q4_0, 130, 512, 3), (D.Q4K, 96, 256, 1)]:
        w = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(dt, n, k, seed=70), (n, k), dt), dev)
        assert w.supports_normed()
        x = torch.randn(1, k, device=dev) * 3; g = torch.rand(k, device=dev) + 0.5
        delta = torch.randn(1, parts * k, device=dev) if parts else None
        # separate kernels: the residual is updated in place
        x_ref = x.clone(); img = ops.ActImage.for_weight(dt, 1, k, dev)
        ops.add_rmsnorm(x_ref, delta, g, 1e-5, None, img)
        want = w.matmul_t(img)
        x_out = torch.full_like(x, float("nan")); got = torch.empty(1, n, device=dev)
        w.matvec_normed(x, delta, g, 1e-5, x_out, got)
        assert torch.equal(x_out, x_ref), (dt.name, k, parts, "residual")
        assert torch.equal(got, want), (dt.name, k, parts, float((got - want).abs().max()))
    g = torch.Generator(device="cpu"); g.manual_seed(12)
    prompt = torch.randint(0, 512, (1, 9), generator=g).to(dev)
    outs = []
    for fused_norm in (True, False):
        m = QLlama(LlamaConfig.tiny(), dev, batch=1, max_seq=64, max_prefill_rows=64, fused_norm=fused_norm)
        m.prefill(prompt)
        toks = m.decode(12)
        outs.append((toks.clone(), m.last_logits.clone()))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])


def test_operand_images_in_the_batched_decoder_are_bit_identical(monkeypatch):
    """Batches above one on Q4_K linears: the norm and the SwiGLU write the integer kernel's operand layout and each linear is
    one kernel; tokens and logits equal those of the planar images."""
    from xn_b200.llama import LlamaConfig, QLlama
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu"); g.manual_seed(14)
    prompt = torch.randint(0, 512, (4, 9), generator=g).to(dev)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("XN_OPERAND_IMAGES", flag)
        m = QLlama(LlamaConfig.tiny(), dev, batch=4, max_seq=64, max_prefill_rows=64)
        m.prefill(prompt)
        toks = m.decode(10)
        outs.append((toks.clone(), m.last_logits.clone()))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_rank(rank, world, port, ret):
    import torch.distributed as dist
    from xn_b200.llama import LlamaConfig, QLlama
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator(device="cpu"); g.manual_seed(7)
        prompt = torch.randint(0, 512, (2, 20), generator=g).to(dev)
        tp = QLlama(LlamaConfig.tiny(), dev, batch=2, max_seq=64, rank=rank, world=world, max_prefill_rows=64)
        lt = tp.prefill(prompt)
        tp.capture_decode()
        dist.barrier()
        toks = tp.decode(6)
        torch.cuda.synchronize(dev)
        late = tp.pg.late_peers()
        single = QLlama(LlamaConfig.tiny(), dev, batch=2, max_seq=64, max_prefill_rows=64)
        ls = single.prefill(prompt)
        single.capture_decode()
        ts = single.decode(6)
        ret[rank] = {"rel": _rel(lt, ls), "same_tokens": bool(torch.equal(toks, ts)), "late": late}
        dist.barrier()
        tp.close()
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_decoder_equals_one_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_tp_rank, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        # the K-sharded o / down projections add their summands in another order, and in prefill each shard's fp16
        # operands carry their own power-of-two scale: logits agree to the prefill path's tolerance, tokens exactly
        assert ret[r]["late"] == 0 and ret[r]["rel"] < 3e-2 and ret[r]["same_tokens"], dict(ret)


def test_gguf_file_round_trip_through_device_handles(tmp_path):
    """Write a GGUF file from device weight handles, map it back, upload whole and as two N-shards: the blocks on
    disk are the canonical ones and the sharded matmuls tile the unsharded result."""
    import numpy as np
    from xn_b200 import gguf, quantized as Q, synth
    from xn_b200.dtypes import GgmlDType as D
    dev = torch.device("cuda", 0)
    specs = [("q4k", D.Q4K, 64, 512), ("q6k", D.Q6K, 32, 256), ("q8_0", D.Q8_0, 64, 128), ("q4_0", D.Q4_0, 96, 64)]
    host = {name: synth.make_weight(dt, n, k, seed=70 + i) for i, (name, dt, n, k) in enumerate(specs)}
    on_dev = [(name, Q.QCudaTensor.from_qtensor(Q.QTensor(host[name], (n, k), dt), dev)) for name, dt, n, k in specs]
    path = tmp_path / "w.gguf"
    with open(path, "wb") as f:
        gguf.write(f, [("general.architecture", gguf.Value(gguf.STRING, "test"))], on_dev)
    c = gguf.Content.read(str(path))
    for name, dt, n, k in specs:
        assert np.array_equal(c.tensor_bytes(name), np.asarray(host[name]).reshape(-1))
        x = torch.randn(3, k, device=dev)
        full = c.upload(name, dev).matmul_t(x)
        parts = [c.upload(name, dev, r, 2).matmul_t(x) for r in range(2)]
        assert torch.equal(torch.cat(parts, dim=-1), full)
