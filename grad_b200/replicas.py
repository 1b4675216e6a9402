"""Host-side mirror of `Replicas` (src/nn/replicas.zig): the data-parallel group of one training or inference job.

One process per GPU (the reference runs one thread per replica, src/nn/trainer.zig:603-612).  The mean of
the gradients is ONE NCCL allreduce over the flat gradient vector on the device (`gb_allreduce_mean`) instead of
two trips through host memory; the barrier with a stop flag that releases waiting replicas when one of them
fails (`wait` / `stop`, replicas.zig:36-53) lives on the rendezvous store, so it works without a GPU.
torch.distributed is only the plumbing that hands rank 0's NCCL id to the others.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from . import abi


class Stopped(RuntimeError):
    """error.Stopped (replicas.zig:41): another replica failed and released the barrier."""


def shard(total: int, count: int, index: int) -> Tuple[int, int]:
    """The slice of `total` items replica `index` of `count` owns: [total*index/count, total*(index+1)/count)
    (replicas.zig:71-72); also how an inference batch is split across GPUs."""
    return total * index // count, total * (index + 1) // count


def flat_grads(shapes: Sequence[Sequence[int]], device, align: int = 4) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """One flat f32 gradient vector with a view per parameter, the layout `gradLen` describes (replicas.zig:95-99):
    the whole model's gradients are then averaged by ONE collective.  Every view starts on a multiple of `align`
    elements (16 bytes), so the contraction kernels can store into it with their vector / TMA stores."""
    offsets, total = [], 0
    for shape in shapes:
        total = (total + align - 1) // align * align
        offsets.append(total)
        n = 1
        for d in shape:
            n *= int(d)
        total += n
    flat = torch.zeros(total, dtype=torch.float32, device=device)
    views = []
    for shape, off in zip(shapes, offsets):
        n = 1
        for d in shape:
            n *= int(d)
        views.append(flat[off:off + n].view(*shape))
    return flat, views


class Replicas:
    def __init__(self, count: int, index: int, device: Optional[int] = None, store=None, timeout_s: float = 60.0):
        self.count, self.index, self.device = count, index, device
        self.timeout_s = timeout_s
        self.store = store if store is not None else (dist.distributed_c10d._get_default_store() if dist.is_initialized() else None)
        self.generation = 0
        self.comm = None
        self.lib = None
        if count > 1 and device is not None:
            self.lib = abi.library()
            ident = (C.c_ubyte * 128)()
            if index == 0:
                abi.check(self.lib.gb_comm_unique_id(ident), "gb_comm_unique_id")
            payload = [bytes(ident)]
            dist.broadcast_object_list(payload, src=0)
            ident = (C.c_ubyte * 128).from_buffer_copy(payload[0])
            comm = C.c_void_p()
            abi.check(self.lib.gb_comm_create(count, index, ident, device, C.byref(comm)), "gb_comm_create")
            self.comm = comm
            abi.check(self.lib.gb_comm_set_timeout(comm, max(1, int(timeout_s * 1000))), "gb_comm_set_timeout")

    # ---- barrier with a stop flag (replicas.zig:36-53) ---------------------------------------------------
    def stop(self):
        if self.store is not None:
            self.store.set("gb_replicas_stopped", "1")
        self._abort()

    def _abort(self):
        if self.comm is not None:
            self.lib.gb_comm_abort(self.comm)

    def _stopped(self) -> bool:
        try:
            return self.store.check(["gb_replicas_stopped"])
        except Exception:
            return False

    def wait(self):
        """Blocks until every replica has called it; raises Stopped if one has called stop().  A replica released by
        the stop flag or by the deadline also aborts its own communicator, so nothing it enqueues later can wait on
        the device for the replica that failed."""
        if self.count == 1:
            return
        if self._stopped():
            self._abort()
            raise Stopped()
        self.generation += 1
        key = f"gb_replicas_gen_{self.generation}"
        arrived = self.store.add(key, 1)
        deadline = time.monotonic() + self.timeout_s
        while arrived < self.count:
            if self._stopped():
                self._abort()
                raise Stopped()
            if time.monotonic() > deadline:
                self._abort()
                raise TimeoutError(f"replica barrier {self.generation}: {arrived} of {self.count} arrived")
            time.sleep(0.001)
            arrived = self.store.add(key, 0)

    # ---- the gradient mean (replicas.zig:57-91) ------------------------------------------------------------
    @staticmethod
    def _span(grads: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
        """The one contiguous f32 range that covers `grads` when they are views into one flat buffer (in order,
        gaps of alignment padding allowed), else None."""
        first = grads[0]
        storage = first.untyped_storage().data_ptr()
        end = first.data_ptr()
        for g in grads:
            if g.untyped_storage().data_ptr() != storage or g.data_ptr() < end or g.data_ptr() - end > 64:
                return None
            end = g.data_ptr() + g.numel() * 4
        count = (end - first.data_ptr()) // 4
        return torch.as_strided(first, (count,), (1,))

    def averageGrads(self, grads: Union[torch.Tensor, Sequence[torch.Tensor]], finish: bool = False, barrier: bool = True):
        """Replaces every gradient, in every replica, by the mean over the replicas; identical bits everywhere.
        The replicas first meet at the barrier (replicas.zig:67), so a replica that has failed releases the others
        with `Stopped` before any of them has enqueued the collective.  A flat f32 tensor, or views into one flat
        buffer (`flat_grads`), are reduced by ONE call like the reference's single flat vector; tensors that live
        in separate allocations are reduced one after the other.  `finish` waits for the result on the host with
        the group's deadline (the bounded form of the barrier after the reduction, replicas.zig:81).  `barrier=False`
        skips the host barrier in front (a store round trip per step) for callers that rely on `finish` and the
        communicator's deadline alone to be released from a replica that failed."""
        if self.count == 1:
            return
        if self.comm is None:
            raise RuntimeError("averageGrads needs a CUDA device: the mean runs over NCCL, there is no host path")
        if barrier:
            self.wait()
        if isinstance(grads, torch.Tensor):
            grads = [grads]
        for g in grads:
            assert g.dtype == torch.float32 and g.is_contiguous()
        span = self._span(grads) if len(grads) > 1 else grads[0].view(-1)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream) if grads[0].is_cuda else None
        for g in ([span] if span is not None else grads):
            self._check(self.lib.gb_allreduce_mean(self.comm, stream, C.c_void_p(g.data_ptr()), g.numel()), "gb_allreduce_mean")
        if finish:
            self._check(self.lib.gb_comm_finish(self.comm, stream), "gb_comm_finish")

    def _check(self, rc: int, where: str):
        if rc == 0:
            return
        if rc in (5, 6):   # GB_ERR_TIMEOUT / GB_ERR_NCCL: the communicator is gone; tell the others
            if self.store is not None:
                self.store.set("gb_replicas_stopped", "1")
            raise Stopped(f"{where}: {abi.STATUS_NAMES.get(rc, rc)}")
        raise abi.GbError(rc, where)

    def close(self):
        if self.comm is not None:
            self.lib.gb_comm_destroy(self.comm)
            self.comm = None
