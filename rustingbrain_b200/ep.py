"""Expert parallelism over the GPUs of one node.

The reference crate is single-device ("no multi-GPU, no distributed training",
README.md:29-31); this module adds the one parallel axis the MoE path offers:
rank ``r`` of ``N`` owns experts ``[r*E/N, (r+1)*E/N)``, the router and the shared
expert are replicated, and rows travel to their expert's owner and back with NCCL
send/recv inside the C library (``moe_ep_*`` in ``include/moe_b200.h``).

``torch.distributed`` is used only as the host channel that hands the NCCL unique
id from rank 0 to the other ranks; the row exchange itself never goes through it.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .moe import MoeConfig, MoeLayer, NetworkError


def exchange_plan(counts_all, rank):
    """Host-side plan of one exchange (``moe_ep_plan``); needs no GPU.

    ``counts_all[s, e]`` = rows rank ``s`` routes to global expert ``e``.  Returns a dict
    with ``send_off`` [E+1], ``recv_row`` [N, E/N], ``local_row0`` / ``local_tiles`` /
    ``local_counts`` [E/N+1] and ``rows`` (padded local total).
    """
    counts_all = np.ascontiguousarray(counts_all, dtype=np.int32)
    N, E = counts_all.shape
    El = E // N
    send_off = np.zeros(E + 1, np.int32)
    recv_row = np.zeros((N, El), np.int32)
    row0 = np.zeros(El + 1, np.int32)
    tiles = np.zeros(El + 1, np.int32)
    cnt = np.zeros(El + 1, np.int32)
    ip = C.POINTER(C.c_int32)
    rows = _lib.lib().moe_ep_plan(counts_all.ctypes.data_as(ip), N, E, rank, send_off.ctypes.data_as(ip),
                                  recv_row.ctypes.data_as(ip), row0.ctypes.data_as(ip), tiles.ctypes.data_as(ip),
                                  cnt.ctypes.data_as(ip))
    if rows < 0:
        raise ValueError("bad exchange-plan arguments")
    return dict(send_off=send_off, recv_row=recv_row, local_row0=row0, local_tiles=tiles, local_counts=cnt[:El],
                rows=int(rows))


class RankMissing(NetworkError):
    """A rank of the group did not arrive within the deadline (nothing was launched)."""


_join_count = 0


def join_ranks(timeout_s: float, tag: str = "moe_ep_join") -> None:
    """Host-side check-in of every rank of the default group, with a deadline.

    Called before the communicator is created (``ncclCommInitRank`` itself has no deadline: a rank that
    never arrives would leave the others inside it for ever) and, optionally, before every step.  Each rank
    adds itself to a counter in the group's key-value store and polls it until every rank is there; a rank
    that is still alone after ``timeout_s`` raises ``RankMissing`` without having touched a GPU, so the
    failure is learnt on the host before the next launch.  Every rank must call it the same number of times.
    """
    import time
    import torch.distributed as dist
    global _join_count
    _join_count += 1
    world = dist.get_world_size()
    if world == 1:
        return
    store = dist.distributed_c10d._get_default_store()
    key = "%s/%d" % (tag, _join_count)
    store.add(key, 1)
    t0 = time.monotonic()
    while True:
        n = store.add(key, 0)
        if n >= world:
            return
        if time.monotonic() - t0 > timeout_s:
            raise RankMissing("Timeout: %d of %d ranks checked in within %.1f s (%s); no collective was started"
                              % (n, world, timeout_s, key))
        time.sleep(0.002)


class ExpertParallelMoe(MoeLayer):
    """A ``MoeLayer`` whose experts are split over the ranks of ``torch.distributed``'s default group.

    ``forward`` / ``forward_train`` / ``backward`` are collectives: every rank calls them
    in the same order, each with its own tokens.  Losses and router gradients are those of
    the concatenated batch, as if one device had seen every rank's tokens.
    """

    def __init__(self, d_model: int, config: MoeConfig, *, precision: str = "bf16", max_tokens: int = 4096,
                 device: int = 0, training: bool = True, capacity_factor: float = 0.0, transport: str = "peer",
                 join_timeout_s: float = 300.0, deadline_s: float = 600.0, step_check_in: bool = False):
        """``join_timeout_s``: how long to wait for every rank before the communicator is created;
        ``deadline_s``: how long a host-side wait behind a collective may take before the group is aborted
        (``moe_ep_set_deadline_ms``; 0 = for ever); ``step_check_in``: also check in on the host before every
        forward pass, so that a rank that left between steps is noticed before the next launch."""
        import torch
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before ExpertParallelMoe is built")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self._join_timeout_s, self._step_check_in = join_timeout_s, step_check_in
        join_ranks(join_timeout_s)
        super().__init__(d_model, config, precision=precision, max_tokens=max_tokens, device=device, training=training,
                         ep_rank=self.rank, ep_size=self.world, ep_capacity_factor=capacity_factor)
        n = 128
        buf = (C.c_uint8 * n)()
        if self.rank == 0:
            self._ck(_lib.lib().moe_ep_unique_id(buf, n))
        on_gpu = dist.get_backend() == "nccl"
        t = torch.tensor(list(buf), dtype=torch.uint8, device=("cuda:%d" % device) if on_gpu else "cpu")
        dist.broadcast(t, 0)
        raw = bytes(t.cpu().tolist())
        self._ck(_lib.lib().moe_ep_init(self._h, raw, n))
        self._ck(_lib.lib().moe_ep_set_deadline_ms(self._h, int(deadline_s * 1000)))
        self.transport = transport
        if transport == "peer":
            # map every rank's receive buffers into this process (CUDA IPC); rows then move by
            # direct stores / loads over NVLink inside the dispatch and combine kernels
            hb = (C.c_uint8 * 256)()
            self._ck(_lib.lib().moe_ep_export_buffers(self._h, hb, 256))
            all_handles = [None] * self.world
            dist.all_gather_object(all_handles, bytes(hb))
            for r, h in enumerate(all_handles):
                self._ck(_lib.lib().moe_ep_import_buffers(self._h, r, h, 256))
        elif transport != "nccl":
            raise ValueError("transport must be 'peer' or 'nccl'")

    def forward_train(self, *args, **kwargs):
        if self._step_check_in:
            join_ranks(self._join_timeout_s, "moe_ep_step")
        return super().forward_train(*args, **kwargs)

    def owned_experts(self):
        el = self.config.num_experts // self.world
        return range(self.rank * el, (self.rank + 1) * el)
