"""N-sharded (tensor-parallel along the output dimension) quantized linears.

The reference has no multi-device code at all (one `Device`, one stream:
xn-core/src/cuda_backend/mod.rs:141-167).  The path shards naturally: every output column is an
independent dot product (k_quants.rs:72-75), so rank r of G holds weight rows
``[r*n/G, (r+1)*n/G)``, every rank quantizes the same activations (bit-identical), and the only
exchange is the gather of the ``[m, n/G]`` output slices.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def shard_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """Rows ``[r0, r1)`` of an ``n``-row weight that rank ``rank`` of ``world`` holds."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"shard {rank} of {world}")
    if n % world:
        raise ValueError(f"n = {n} does not divide over {world} shards")
    per = n // world
    return rank * per, (rank + 1) * per


def gather_columns(y_local: torch.Tensor, world: int, group: Optional[dist.ProcessGroup] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather ``[.., n/G]`` slices into ``[.., n]`` on every rank (rank r's slice lands in columns
    ``[r*n/G, (r+1)*n/G)``).  One collective; for a single row the gathered buffer already is the result."""
    if world == 1:
        return y_local
    lead, nl = y_local.shape[:-1], y_local.shape[-1]
    flat = y_local.reshape(-1, nl).contiguous()
    m = flat.shape[0]
    buf = out if out is not None else torch.empty((world, m, nl), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(buf.view(world * m, nl), flat, group=group)
    if m == 1:
        return buf.view(*lead, world * nl)
    return buf.permute(1, 0, 2).reshape(*lead, world * nl)


class ShardedQLinear:
    """A quantized linear whose weight rows are split over the ranks of a process group; ``forward``
    returns the full ``[.., n]`` output on every rank."""

    def __init__(self, local_linear, n_total: int, world: int, group: Optional[dist.ProcessGroup] = None):
        self.local, self.n_total, self.world, self.group = local_linear, n_total, world, group

    @classmethod
    def from_qtensor(cls, qt, device, rank: int, world: int, group: Optional[dist.ProcessGroup] = None) -> "ShardedQLinear":
        from .quantized import QCudaLinear, QCudaTensor
        n, _ = qt.shape()
        shard_rows(n, rank, world)  # validates
        return cls(QCudaLinear(QCudaTensor.from_qtensor(qt, device, shard_rank=rank, shard_count=world)), n, world, group)

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        return gather_columns(self.local.forward(xs), self.world, self.group)

    __call__ = forward


class _DeviceBuffer:
    """A view of library-owned device memory that torch can wrap without copying."""

    def __init__(self, ptr: int, shape: tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": shape, "typestr": typestr, "version": 2, "strides": None}


_TYPESTR = {torch.float32: "<f4", torch.float16: "<f2", torch.bfloat16: "<i2"}  # bf16 travels as 16-bit words and is re-viewed


class PeerGather:
    """The ranks' gathered-output slots (``xnq_comm``): rank r's matmul kernel stores its output
    columns into the same slot of every rank over NVLink, so there is no collective call. ``slot_elems``
    is the largest ``m * n_total`` any gather will produce; handles travel over ``group``."""

    def __init__(self, device: torch.device, rank: int, world: int, slot_elems: int, nslots: int = 2,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes

        from . import _lib
        from .quantized import init
        init(device)
        self.device, self.rank, self.world, self.nslots, self.group = device, rank, world, nslots, group
        self._L = _lib.lib()
        self._h = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(self._L.xnq_comm_create(rank, world, slot_elems * 4, nslots, ctypes.byref(self._h)))
            mine = ctypes.create_string_buffer(64)
            _lib.check(self._L.xnq_comm_ipc_handle(self._h, mine))
            if world > 1:
                handles = [None] * world
                dist.all_gather_object(handles, bytes(mine.raw), group=group)
                error = None
                try:
                    _lib.check(self._L.xnq_comm_connect(self._h, ctypes.create_string_buffer(b"".join(handles), 64 * world)))
                except _lib.XnqError as e:   # e.g. peer mappings are not permitted here: every rank has to learn of it
                    error = e
                # nobody stores into a peer before every peer has mapped everybody; the same collective tells all
                # ranks whether some rank could not map its peers, so that none is left waiting for the others
                ok = torch.tensor([0 if error else 1], device=device if dist.get_backend(group) == "nccl" else "cpu")
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    self._L.xnq_comm_free(self._h)
                    self._h = None
                    raise RuntimeError(f"peer mappings could not be set up on every rank ({error or 'another rank failed'})")
        self._next = 0
        self.slot_elems = slot_elems

    def set_deferred(self, deferred: bool) -> None:
        """Deferred waits: gathers publish and retire; ``wait()`` awaits the peers' columns of all gathers issued so far and
        must lie between a gather and the first reader of its slot (xnq_comm_set_deferred / xnq_comm_wait)."""
        from . import _lib
        _lib.check(self._L.xnq_comm_set_deferred(self._h, 1 if deferred else 0))

    def wait(self) -> None:
        from . import _lib
        from .quantized import _stream_ptr
        with torch.cuda.device(self.device):
            _lib.check(self._L.xnq_comm_wait(self._h, _stream_ptr(self.device)))

    def next_slot(self) -> int:
        s = self._next
        self._next = (s + 1) % self.nslots
        return s

    def matmul_t(self, w, lhs: torch.Tensor, slot: Optional[int] = None, parts: bool = False) -> torch.Tensor:
        """``lhs @ W^T`` for the N-sharded ``w`` (a ``QCudaTensor`` shard), gathered: ``(.., n_total)`` on
        every rank, living in one of this object's slots until that slot is named again. With ``parts`` the
        weight is a whole-N one (a K-shard fed with this rank's input slice) and the result is
        ``(.., world * n)``: every rank's summand side by side, for the consumer to add."""
        import ctypes

        from . import _lib
        from .quantized import _TORCH_TO_XNQ, _stream_ptr
        image = hasattr(lhs, "act_dtype")   # an ActImage: activations quantized ahead of the call
        if (lhs.k if image else lhs.shape[-1]) != w.k:
            raise ValueError(f"cuda quantized matmul: input does not match weight (n={w.n}, k={w.k})")
        if image:
            x, m, xdt, ldx, ydt, lead = lhs, lhs.m, _lib.XNQ_ACT_IMAGE, 0, torch.float32, (lhs.m,)
        else:
            x = lhs.reshape(-1, w.k)
            if x.stride(-1) != 1 or (x.shape[0] > 1 and x.stride(0) < w.k):
                x = x.contiguous()
            m = x.shape[0]
            xdt, ldx = int(_TORCH_TO_XNQ[x.dtype]), (x.stride(0) if m > 1 else w.k)
            ydt = lhs.dtype if lhs.dtype in _TYPESTR else torch.float32
            lead = lhs.shape[:-1]
        slot = self.next_slot() if slot is None else slot
        ws = w.workspace(m)
        out = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self._L.xnq_matmul_t_gather(w._h, self._h, slot, 1 if parts else 0, ctypes.c_void_p(x.data_ptr()), xdt, m, ldx,
                                                  int(_TORCH_TO_XNQ[ydt]), ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(self.device),
                                                  ctypes.byref(out)))
        nt = w.n * self.world if parts else w.n_total
        y = torch.as_tensor(_DeviceBuffer(out.value, (m, nt), _TYPESTR[ydt]), device=self.device)
        if ydt is torch.bfloat16:
            y = y.view(torch.bfloat16)
        return y.view(*lead, nt)

    def gather(self, y_local: torch.Tensor, slot: Optional[int] = None) -> torch.Tensor:
        """All-gather ``(.., n_local)`` blocks that each rank already holds into ``(.., world * n_local)``."""
        import ctypes

        from . import _lib
        from .quantized import _TORCH_TO_XNQ, _stream_ptr
        if self.world == 1:
            return y_local
        nl = y_local.shape[-1]
        src = y_local.reshape(-1, nl)
        if src.stride(-1) != 1:
            src = src.contiguous()
        m = src.shape[0]
        slot = self.next_slot() if slot is None else slot
        out = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self._L.xnq_comm_gather(self._h, slot, ctypes.c_void_p(src.data_ptr()), int(_TORCH_TO_XNQ[src.dtype]), m, nl,
                                               src.stride(0) if m > 1 else nl, _stream_ptr(self.device), ctypes.byref(out)))
        y = torch.as_tensor(_DeviceBuffer(out.value, (m, nl * self.world), _TYPESTR[src.dtype]), device=self.device)
        if src.dtype is torch.bfloat16:
            y = y.view(torch.bfloat16)
        return y.view(*y_local.shape[:-1], nl * self.world)

    def late_peers(self) -> int:
        import ctypes

        from . import _lib
        bits = ctypes.c_uint()
        with torch.cuda.device(self.device):
            _lib.check(self._L.xnq_comm_status(self._h, ctypes.byref(bits)))
        return bits.value

    def close(self):
        if self._h:
            self._L.xnq_comm_free(self._h)
            self._h = None
