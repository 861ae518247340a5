"""N-sharded matmul whose kernels store their output columns into every rank's buffer (xnq_comm_*,
xnq_matmul_t_gather): one rank on one GPU, and two ranks on two GPUs when the machine has them. The
checker is the CPU oracle on the unsharded weight."""
import os
import socket

import numpy as np
import pytest
import torch

from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

pytestmark = pytest.mark.gpu

CASES = [(D.Q4K, 512, 1024, 1), (D.Q6K, 384, 512, 1), (D.Q8_0, 256, 4096, 1), (D.Q4_0, 320, 512, 1),   # decode kernel stores remotely itself
         (D.Q4K, 256, 1024, 5), (D.Q8_0, 256, 8192, 1), (D.Q4K, 256, 512, 40)]                         # pushed by the copy kernel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_rank(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from xn_b200 import quantized as Q
        from xn_b200.parallel import PeerGather, shard_rows
        Q.init(dev)
        pg = PeerGather(dev, rank, world, slot_elems=40 * 512, nslots=3)
        bad = []
        for dt, n, k, m in CASES:
            full = synth.make_weight(dt, n, k, seed=900)
            r0, r1 = shard_rows(n, rank, world)
            w = Q.QCudaTensor.from_rows(dt, synth.make_weight(dt, n, k, seed=900, rows=(r0, r1)), n, k, r0, r1 - r0, dev)
            x = synth.make_activation(m, k, seed=901)
            ref = O.matmul(int(dt), x, full, n, threads=4)
            xd = torch.from_numpy(x).to(dev)
            for rep in range(3):  # the same gather again: epochs advance, slots rotate
                y = pg.matmul_t(w, xd).float().cpu().numpy()
                tol = (2e-3 if m <= 16 else 1e-2) * max(1.0, float(np.sqrt((ref ** 2).mean())))
                err = float(np.abs(y - ref).max())
                if y.shape != (m, n) or not err <= tol:
                    bad.append((dt.name, n, k, m, rep, err, tol))
            dist.barrier()  # a weight is freed only after every rank has finished with its gathers
        # row-parallel: each rank holds a K-shard (whole-N weight over its own input slice); the slot receives the summands
        dt, n, k, m = D.Q4K, 256, 1024 * world, 1
        full = synth.make_weight(dt, n, k, seed=903)
        x = synth.make_activation(m, k, seed=904)
        ref = O.matmul(int(dt), x, full, n, threads=4)
        kl = k // world
        rb = dt.row_bytes(k) // world
        shard = np.ascontiguousarray(full.reshape(n, dt.row_bytes(k))[:, rank * rb:(rank + 1) * rb])
        w = Q.QCudaTensor.from_rows(dt, shard, n, kl, 0, n, dev)
        xd = torch.from_numpy(np.ascontiguousarray(x[:, rank * kl:(rank + 1) * kl])).to(dev)
        y = pg.matmul_t(w, xd, parts=True)
        got = y.view(m, world, n).sum(1).cpu().numpy()
        if y.shape != (m, world * n) or not float(np.abs(got - ref).max()) <= 2e-3 * max(1.0, float(np.sqrt((ref ** 2).mean()))):
            bad.append(("parts", float(np.abs(got - ref).max())))
        dist.barrier()
        # graph replay: epochs are device-side, so a captured pair of gathers can be replayed
        dt, n, k = D.Q4K, 512, 1024
        r0, r1 = shard_rows(n, rank, world)
        w = Q.QCudaTensor.from_rows(dt, synth.make_weight(dt, n, k, seed=900, rows=(r0, r1)), n, k, r0, r1 - r0, dev)
        x = synth.make_activation(1, k, seed=902)
        ref = O.matmul(int(dt), x, synth.make_weight(dt, n, k, seed=900), n, threads=4)
        xd = torch.from_numpy(x).to(dev)
        pg.matmul_t(w, xd, slot=1); pg.matmul_t(w, xd, slot=2)
        torch.cuda.synchronize(dev)
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                y0 = pg.matmul_t(w, xd, slot=0)
                y1 = pg.matmul_t(w, xd, slot=1)
        for rep in range(4):
            y0.zero_(); y1.zero_()
            torch.cuda.synchronize(dev)
            dist.barrier()
            g.replay()
            torch.cuda.synchronize(dev)
            for y in (y0, y1):
                err = float(np.abs(y.cpu().numpy() - ref).max())
                if not err <= 2e-3 * max(1.0, float(np.sqrt((ref ** 2).mean()))):
                    bad.append(("graph", rep, err))
            dist.barrier()
        late = pg.late_peers()
        import ctypes
        from xn_b200 import _lib
        bits = ctypes.c_uint(123)
        _lib.check(_lib.lib().xnq_device_status(ctypes.byref(bits)))
        status = bits.value
        dist.barrier()
        pg.close()
        ret[rank] = {"bad": bad, "late": late, "status": status}
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_kernel_side_gather_matches_the_unsharded_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_run_rank, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r]["bad"] == [] and ret[r]["late"] == 0 and ret[r]["status"] == 0, dict(ret)


def test_consecutive_gathers_on_one_slot_are_refused():
    from xn_b200 import _lib, quantized as Q
    from xn_b200.parallel import PeerGather
    dev = torch.device("cuda", 0)
    Q.init(dev)
    pg = PeerGather(dev, 0, 1, slot_elems=1024)
    w = Q.QCudaTensor.from_rows(D.Q4K, synth.make_weight(D.Q4K, 64, 256, seed=1), 64, 256, 0, 64, dev)
    x = torch.zeros((1, 256), device=dev)
    pg.matmul_t(w, x, slot=0)
    with pytest.raises(_lib.XnqError):
        pg.matmul_t(w, x, slot=0)
    with pytest.raises(_lib.XnqError):
        pg.matmul_t(w, torch.zeros((32, 256), device=dev), slot=1)  # 32 * 64 elements do not fit a 1024-element slot
    pg.close()
