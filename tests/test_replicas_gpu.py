"""The gradient mean over NCCL on two GPUs (tests/replicas.zig:60-103: every replica ends with identical bits that
match the mean of the per-replica gradients).  Needs two CUDA devices; child processes, one per GPU."""
import multiprocessing as mp
import os
import socket
import traceback

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, queue):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
        import torch
        import torch.distributed as dist

        from grad_b200.replicas import Replicas, flat_grads

        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)   # plumbing only: the mean itself runs through gb_allreduce_mean
        group = Replicas(world, rank, device=rank)
        gen = torch.Generator(device="cuda").manual_seed(100 + rank)
        # the MLP's gradients as views of one flat vector (one collective) and one tensor in its own allocation
        flat, views = flat_grads([(784, 128), (128,), (128, 10), (10,)], "cuda")
        flat.copy_(torch.randn(flat.numel(), generator=gen, device="cuda"))
        lone = torch.randn(3228737, generator=gen, device="cuda")      # the character Transformer's gradient length
        grads = [flat, lone]
        before = [g.cpu().numpy().copy() for g in grads]
        group.averageGrads(views)
        group.averageGrads(lone, finish=True)
        torch.cuda.synchronize()
        group.wait()
        queue.put((rank, "ok", before, [g.cpu().numpy() for g in grads]))
        group.close()
        dist.destroy_process_group()
    except Exception:
        queue.put((rank, "error", traceback.format_exc(), None))


def test_average_grads_is_the_mean_and_identical_on_both_replicas():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted((queue.get(timeout=300) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in results] == ["ok", "ok"], results
    from oracle import binding as orc

    for i in range(2):
        a, b = results[0][3][i], results[1][3][i]
        assert np.array_equal(a, b)                      # identical bits on every replica (replicas.zig:56)
        stacked = np.stack([results[0][2][i].ravel(), results[1][2][i].ravel()])
        want = orc.average_grads(stacked)[0].reshape(a.shape)
        np.testing.assert_allclose(a, want, rtol=1e-6, atol=1e-7)
