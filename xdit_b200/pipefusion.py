"""PipeFusion patch hand-off between pipeline stages, with the interface of the reference's
``PipelineGroupCoordinator`` (``xfuser/core/distributed/group_coordinator.py:915-985``):
``pipeline_isend``, ``add_pipeline_recv_task``, ``recv_next``, ``get_pipeline_recv_data``,
``pipeline_send`` / ``pipeline_recv``, and the stage loop of the asynchronous pipeline
(``xfuser/model_executor/pipelines/pipeline_pixart_sigma.py:474-560``).

In PipeFusion the token sequence is cut into patches that travel through the pipeline stages one after
the other; a stage works on patch ``p`` of denoising step ``i`` while the next stage still works on
patch ``p-1``, and attention inside a stage reads a per-layer K/V buffer whose rows for the other patches
are one step stale (``xdit_b200.cache_manager``).  The reference receives every patch into a separate
buffer (``recv_buffer[name][idx]``) and joins the patches with ``torch.cat`` at the end of the run.  Here
the patches of a stage's input live in ONE persistent activation buffer ``[B, S, C]`` (patch ``p`` =
rows ``[start_p, end_p)``): each receive is posted ahead of time straight into its rows, so a patch is in
place when it arrives, the full-sequence tensor exists at all times without a concatenation, and the
stale-KV rows of the same token range are overwritten by the layer's own producer kernel.

One receive is kept in flight ahead of the patch being computed, like the reference's
``recv_next`` / ``get_pipeline_recv_data`` pair; sends are asynchronous and their requests are kept until
the buffer they read may be reused.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class PatchPipe:
    """The link of one pipeline stage to its neighbours inside a pipeline-parallel group."""

    def __init__(self, group, patch_rows: Sequence[int], batch: int, channels: int, dtype, device):
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank_in_group = dist.get_rank(group)
        nxt, prv = (self.rank_in_group + 1) % self.world_size, (self.rank_in_group - 1) % self.world_size
        self.next_rank = dist.get_global_rank(group, nxt) if group is not None else nxt
        self.prev_rank = dist.get_global_rank(group, prv) if group is not None else prv
        # With two stages both directions join the same pair of ranks; a send and a receive posted on one
        # communicator at the same time can wait for each other, so each direction gets a communicator of
        # its own (the reference does the same, group_coordinator.py:966-984).
        self._send_group = self._recv_group = group
        if self.world_size == 2:
            ranks = [dist.get_global_rank(group, i) if group is not None else i for i in range(2)]
            pair = [dist.new_group(ranks), dist.new_group(ranks)]
            self._send_group = pair[self.rank_in_group % 2]
            self._recv_group = pair[(self.rank_in_group + 1) % 2]
        self.patch_rows = list(patch_rows)
        self.starts = [0]
        for n in self.patch_rows:
            self.starts.append(self.starts[-1] + n)
        self.batch, self.channels = batch, channels
        # persistent input activations of this stage: [B, S, C]; with B == 1 a patch's rows are contiguous
        # and are received in place, otherwise each patch has its own contiguous slot
        self.in_place = batch == 1
        if self.in_place:
            self.buffer = torch.zeros(batch, self.starts[-1], channels, dtype=dtype, device=device)
            self.slots = [self.buffer[:, self.starts[i]:self.starts[i + 1]] for i in range(len(self.patch_rows))]
        else:
            self.buffer = None
            self.slots = [torch.zeros(batch, n, channels, dtype=dtype, device=device) for n in self.patch_rows]
        if len(self.patch_rows) == 1:
            # one patch: the next step's patch would land in the rows that are being worked on, so two
            # slots alternate instead
            self.in_place = False
            self.slots = [torch.zeros(batch, self.patch_rows[0], channels, dtype=dtype, device=device) for _ in range(2)]
        self._single = len(self.patch_rows) == 1
        self._posted = 0
        self.recv_tasks_queue: List[int] = []
        self.receiving_tasks: List[tuple] = []
        self._sends: List[tuple] = []

    # ------------------------------------------------------------------ stage position
    @property
    def is_first_stage(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last_stage(self) -> bool:
        return self.rank_in_group == self.world_size - 1

    # ------------------------------------------------------------------ receive side
    def add_pipeline_recv_task(self, idx: int) -> None:
        """Queue the receive of patch ``idx`` (``group_coordinator.py:933-935``)."""
        self.recv_tasks_queue.append(idx)

    def recv_next(self) -> None:
        """Post the next queued receive, straight into the patch's rows (``group_coordinator.py:937-946``)."""
        if len(self.recv_tasks_queue) == 0:
            raise ValueError("No more tasks to receive")
        idx = self.recv_tasks_queue.pop(0)
        slot = self.slots[self._posted % 2] if self._single else self.slots[idx]
        self._posted += 1
        req = dist.irecv(slot, src=self.prev_rank, group=self._recv_group)
        self.receiving_tasks.append((req, idx, slot))

    def get_pipeline_recv_data(self, idx: int) -> torch.Tensor:
        """Wait for the oldest posted receive, which must be patch ``idx``; returns the patch's rows
        (a view of the persistent buffer; ``group_coordinator.py:948-961``)."""
        assert len(self.receiving_tasks) > 0, "No tasks to receive, call add_pipeline_recv_task first"
        req, got, slot = self.receiving_tasks.pop(0)
        req.wait()
        assert got == idx, "Received tensor does not match the requested"
        return slot

    def pipeline_recv(self, idx: int) -> torch.Tensor:
        """Blocking receive of patch ``idx`` (``group_coordinator.py:925-931``)."""
        dist.irecv(self.slots[idx], src=self.prev_rank, group=self._recv_group).wait()
        return self.slots[idx]

    # ------------------------------------------------------------------ send side
    def pipeline_isend(self, tensor: torch.Tensor, segment_idx: int = -1) -> None:
        """Asynchronous send of a patch to the next stage (``group_coordinator.py:906-913``).  The request
        (and the tensor) are kept until ``flush_sends`` or until two newer sends have been issued."""
        tensor = tensor.contiguous()
        req = dist.isend(tensor, dst=self.next_rank, group=self._send_group)
        self._sends.append((req, tensor))
        while len(self._sends) > 2 * max(1, len(self.patch_rows)):
            old, _ = self._sends.pop(0)
            old.wait()

    def pipeline_send(self, tensor: torch.Tensor, segment_idx: int = -1) -> None:
        tensor = tensor.contiguous()
        dist.isend(tensor, dst=self.next_rank, group=self._send_group).wait()

    def flush_sends(self) -> None:
        for req, _ in self._sends:
            req.wait()
        self._sends = []

    # ------------------------------------------------------------------ the full sequence
    def full_sequence(self) -> torch.Tensor:
        """All patches as one ``[B, S, C]`` tensor: the persistent buffer itself when ``B == 1`` (the
        reference concatenates, ``pipeline_pixart_sigma.py:563``)."""
        if self.in_place:
            return self.buffer
        if self._single:
            return self.slots[(self._posted - 1) % 2]
        return torch.cat(self.slots, dim=1)


def run_async_steps(pipe: PatchPipe, stage_forward: Callable[[torch.Tensor, int, int], torch.Tensor], num_steps: int,
                    runtime_state, first_input: Optional[List[torch.Tensor]] = None,
                    finish_patch: Optional[Callable[[torch.Tensor, int, int], torch.Tensor]] = None
                    ) -> Optional[List[torch.Tensor]]:
    """The stage loop of PipeFusion's asynchronous phase (``pipeline_pixart_sigma.py:500-545``), for every
    stage of the pipeline.

    ``stage_forward(x, step, patch_idx)`` runs this stage's layers on one patch (attention in patch mode:
    ``runtime_state.patch_mode`` is set and ``pipeline_patch_idx`` is advanced here).  The first stage
    starts step 0 from ``first_input`` (one tensor per patch) and later steps from what the last stage
    sends round; the last stage applies ``finish_patch`` (the scheduler step) and returns the final
    patches of the last step.
    """
    P = len(pipe.patch_rows)
    runtime_state.set_patched_mode(True)
    for i in range(num_steps):
        for p in range(P):
            if not (pipe.is_first_stage and i == 0):
                pipe.add_pipeline_recv_task(p)
    last = [None] * P if pipe.is_last_stage else None
    first_async_recv = True
    for i in range(num_steps):
        for p in range(P):
            if pipe.is_first_stage and i == 0:
                x = first_input[p]
            else:
                if first_async_recv:
                    pipe.recv_next()
                    first_async_recv = False
                x = pipe.get_pipeline_recv_data(p)
            runtime_state.pipeline_patch_idx = p
            y = stage_forward(x, i, p)
            if pipe.is_last_stage:
                if finish_patch is not None:
                    y = finish_patch(y, i, p)
                last[p] = y
                if i != num_steps - 1:
                    pipe.pipeline_isend(y, segment_idx=p)
            else:
                pipe.pipeline_isend(y, segment_idx=p)
            if not (pipe.is_first_stage and i == 0):
                if not (i == num_steps - 1 and p == P - 1):
                    pipe.recv_next()
    pipe.flush_sends()
    runtime_state.set_patched_mode(False)
    return last
