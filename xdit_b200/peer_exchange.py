"""Ulysses exchange by direct stores into the peers' memory.

The reference (and this package's default path) moves the head <-> sequence re-layout through NCCL
all-to-all collectives: pack into a send buffer, collective, attention, pack, collective
(``xfuser/model_executor/layers/usp.py:96-150``).  Behind NVSwitch every peer's HBM is one hop away, so
the two kernels that already touch every byte can do the moving themselves:

* the pack kernel stores each peer's block straight into that peer's receive buffer
  (``xdit_ulysses_pack_peers``): no send buffer, no collective, no receive copy;
* the attention kernel's epilogue stores every query segment's rows straight into the ``[B, s, H, D]``
  output buffer of the rank those rows belong to (``xdit_attn_params.out_segments``): the return
  collective and the head-merge re-layout in front of the output projection are gone, and the transfer
  overlaps the arithmetic tile by tile.

Only plain stores to peer-mapped memory are used (no broadcast forms, no loads from peers, no library
kernel is handed a peer pointer); every kernel reads local memory only.  After each of the two kernels the ranks meet
in ``xdit_peer_barrier``: one warp per rank stores the rank's barrier count into every peer's flag array
and waits, with a time limit, until all counts have arrived in its own (a few microseconds; a one-element
NCCL all-reduce in the same place measured tens).  A wait that runs out sets the device's attention status
words, so the next attention call raises instead of computing on incomplete data.

Buffers are allocated once per process group with ``cudaMalloc`` and shared through CUDA IPC handles
(``xdit_peer_alloc`` / ``xdit_peer_open``); they grow (a collective re-allocation) if a later call needs
more.  Results are views of a persistent buffer that alternates between two slots: a returned tensor stays
valid until the second-next call on the same group.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from . import ops

_ENABLED = False
_RING = False
_MIN_BYTES = 0
_MAX_BYTES = 1 << 62
_exchanges: Dict[int, "PeerExchange"] = {}


def enable(on: bool = True, min_bytes: int = 0, max_bytes: int = 1 << 62, ring: Optional[bool] = None) -> None:
    """Switch the direct-store exchange on for Ulysses-only calls whose per-rank send volume lies in
    ``[min_bytes, max_bytes]`` (other calls keep the NCCL path).  ``ring`` (default: the same as ``on``)
    switches the ring K/V rotation from NCCL send/recv to copy-engine transfers into the next rank's buffer."""
    global _ENABLED, _RING, _MIN_BYTES, _MAX_BYTES
    _ENABLED, _MIN_BYTES, _MAX_BYTES = bool(on), int(min_bytes), int(max_bytes)
    _RING = bool(on) if ring is None else bool(ring)


def ring_enabled() -> bool:
    return _RING


def enabled_for(nbytes: int) -> bool:
    return _ENABLED and _MIN_BYTES <= nbytes <= _MAX_BYTES


class PeerExchange:
    OUT_SLOTS = 2

    def __init__(self, group, in_bytes: int, out_bytes: int, device):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        align = lambda n: (int(n) + 255) // 256 * 256
        self.in_bytes, self.out_bytes = align(in_bytes), align(out_bytes)
        self.flag_off = self.in_bytes + self.OUT_SLOTS * self.out_bytes
        total = self.flag_off + 256  # flag words of the barrier: one per rank, at the end of the buffer
        self.ptr, handle, self.local = ops.peer_alloc(total, self.device)
        self.local[self.flag_off:].zero_()
        self._epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.peer_ptr = [self.ptr if r == self.rank else ops.peer_open(handles[r], self.device)
                         for r in range(self.world)]
        self._slot = 0
        dist.barrier(group=group)  # nobody stores into a buffer before every rank has mapped (and zeroed) it

    # receive buffer of the input exchange: one slot (the next call's stores come after this call's reads,
    # see sync())
    def in_local(self, dtype) -> torch.Tensor:
        return self.local[:self.in_bytes].view(dtype)

    def in_peers(self) -> List[int]:
        return list(self.peer_ptr)

    def next_out_slot(self) -> int:
        self._slot = (self._slot + 1) % self.OUT_SLOTS
        return self._slot

    def out_local(self, slot: int, dtype) -> torch.Tensor:
        off = self.in_bytes + slot * self.out_bytes
        return self.local[off:off + self.out_bytes].view(dtype)

    def out_peers(self, slot: int) -> List[int]:
        off = self.in_bytes + slot * self.out_bytes
        return [p + off for p in self.peer_ptr]

    def sync(self) -> None:
        """Every rank's work queued before this point on the current stream has finished before any rank's
        work queued after it starts (``xdit_peer_barrier`` on the current stream)."""
        ops.peer_barrier([p + self.flag_off for p in self.peer_ptr], self.ptr + self.flag_off, self._epoch,
                         self.rank, self.device)

    def close(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for r, p in enumerate(self.peer_ptr):
            if r != self.rank:
                ops.peer_close(p)
        self.local = None
        ops.peer_free(self.ptr)


def get(group, in_bytes: int, out_bytes: int, device) -> PeerExchange:
    """The exchange of ``group``, created or enlarged on demand (collective: every rank of the group makes
    the same call with the same sizes, which holds for the symmetric shards of sequence parallelism)."""
    key = id(group)
    ex = _exchanges.get(key)
    if ex is None or ex.in_bytes < in_bytes or ex.out_bytes < out_bytes:
        if ex is not None:
            in_bytes, out_bytes = max(in_bytes, ex.in_bytes), max(out_bytes, ex.out_bytes)
            ex.close()
        ex = _exchanges[key] = PeerExchange(group, in_bytes, out_bytes, device)
    return ex


def close_all() -> None:
    for ex in list(_exchanges.values()):
        ex.close()
    _exchanges.clear()
