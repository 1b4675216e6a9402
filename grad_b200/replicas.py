"""Host-side mirror of `Replicas` (src/nn/replicas.zig): the data-parallel group of one training or inference job.

One process per GPU (the reference runs one thread per replica, src/nn/trainer.zig:603-612).  The mean of
the gradients goes over NCCL on the device buffers (`gb_allreduce_mean`) instead of through host memory;
the barrier with a stop flag that releases waiting replicas when one of them fails (`wait` / `stop`,
replicas.zig:36-53) lives on the rendezvous store, so it works without a GPU.  torch.distributed is only the
plumbing that hands rank 0's NCCL id to the others.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import abi


class Stopped(RuntimeError):
    """error.Stopped (replicas.zig:41): another replica failed and released the barrier."""


def shard(total: int, count: int, index: int) -> Tuple[int, int]:
    """The slice of `total` items replica `index` of `count` owns: [total*index/count, total*(index+1)/count)
    (replicas.zig:71-72); also how an inference batch is split across GPUs."""
    return total * index // count, total * (index + 1) // count


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

    # ---- barrier with a stop flag (replicas.zig:36-53) ---------------------------------------------------
    def stop(self):
        if self.store is not None:
            self.store.set("gb_replicas_stopped", "1")
        if self.comm is not None:
            self.lib.gb_comm_abort(self.comm)

    def _stopped(self) -> bool:
        try:
            return self.store.check(["gb_replicas_stopped"])
        except Exception:
            return False

    def wait(self):
        """Blocks until every replica has called it; raises Stopped if one has called stop()."""
        if self.count == 1:
            return
        if self._stopped():
            raise Stopped()
        self.generation += 1
        key = f"gb_replicas_gen_{self.generation}"
        arrived = self.store.add(key, 1)
        deadline = time.monotonic() + self.timeout_s
        while arrived < self.count:
            if self._stopped():
                raise Stopped()
            if time.monotonic() > deadline:
                raise TimeoutError(f"replica barrier {self.generation}: {arrived} of {self.count} arrived")
            time.sleep(0.001)
            arrived = self.store.add(key, 0)

    # ---- the gradient mean (replicas.zig:57-91) ------------------------------------------------------------
    def averageGrads(self, grads: Sequence[torch.Tensor]):
        """Replaces every gradient, in every replica, by the mean over the replicas; identical bits everywhere.
        One flat f32 device tensor is reduced in place; several tensors are reduced one after the other."""
        if self.count == 1:
            return
        if self.comm is None:
            raise RuntimeError("averageGrads needs a CUDA device: the mean runs over NCCL, there is no host path")
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for g in grads:
            assert g.is_cuda and g.dtype == torch.float32 and g.is_contiguous()
            rc = self.lib.gb_allreduce_mean(self.comm, stream, C.c_void_p(g.data_ptr()), g.numel())
            if rc != 0:
                raise Stopped() if rc == 6 else abi.GbError(rc, "gb_allreduce_mean")

    def close(self):
        if self.comm is not None:
            self.lib.gb_comm_destroy(self.comm)
            self.comm = None
