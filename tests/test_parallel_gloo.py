"""World-size-2 (and 4) CPU ranks over gloo: the N-sharding host logic. Each rank computes its slice
with the CPU oracle (the test's stand-in for the device kernel), gathers, and must reproduce the
unsharded result exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dt, n, k, m, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from xn_b200.parallel import gather_columns, shard_rows
        r0, r1 = shard_rows(n, rank, world)
        w_local = synth.make_weight(D(dt), n, k, seed=500, rows=(r0, r1))          # only this rank's rows are ever generated
        x = synth.make_activation(m, k, seed=501)                                  # replicated input
        y_local = torch.from_numpy(O.matmul(dt, x, w_local, r1 - r0, threads=1))
        y = gather_columns(y_local, world)
        full = O.matmul(dt, x, synth.make_weight(D(dt), n, k, seed=500), n, threads=1)
        ok = bool(np.array_equal(y.numpy(), full)) and tuple(y.shape) == (m, n)
        y3 = gather_columns(y_local.reshape(1, m, -1), world)                      # leading dims survive
        ok = ok and tuple(y3.shape) == (1, m, n) and bool(np.array_equal(y3.numpy()[0], full))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("dt,m", [(int(D.Q4K), 1), (int(D.Q8_0), 3)])
def test_sharded_rows_gather_to_the_unsharded_result(world, dt, m):
    n, k = 64 * world, 512
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), dt, n, k, m, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_shard_rows_rejects_bad_splits():
    from xn_b200.parallel import shard_rows
    assert shard_rows(128256, 3, 8) == (48096, 64128)
    with pytest.raises(ValueError):
        shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def test_decoder_config_weight_bytes_match_the_published_layer_arithmetic():
    """32 layers x 218,103,808 Q4_K parameters (122,683,392 B) + a 32000 x 4096 Q6_K head (107,520,000 B)."""
    from xn_b200.llama import LlamaConfig
    c = LlamaConfig.llama_7b()
    assert c.weight_bytes_per_step() == 32 * 122_683_392 + 107_520_000 == 4_033_388_544
