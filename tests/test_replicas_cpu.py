"""Host logic of the multi-GPU paths with two gloo ranks on the CPU: batch sharding, the barrier and its stop
flag (tests/replicas.zig:105-118: a failing replica must release the others), rank-0 id hand-off.  The
gradient mean itself runs over NCCL and is covered by tests/test_replicas_gpu.py."""
import multiprocessing as mp
import os
import socket
import traceback

import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, queue):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        import torch.distributed as dist

        from grad_b200.replicas import Replicas, Stopped, shard

        dist.init_process_group("gloo", rank=rank, world_size=world)
        group = Replicas(world, rank, device=None, timeout_s=20)
        if scenario == "barrier":
            for _ in range(3):
                group.wait()
            payload = [b"id-from-rank-0" if rank == 0 else None]
            dist.broadcast_object_list(payload, src=0)
            queue.put((rank, "ok", payload[0], shard(100, world, rank), shard(4096, world, rank)))
        elif scenario == "stop":
            group.wait()
            if rank == 1:
                group.stop()            # this replica fails between steps
                queue.put((rank, "stopped-others"))
            else:
                try:
                    group.wait()
                    queue.put((rank, "not released"))
                except Stopped:
                    queue.put((rank, "released"))
        dist.destroy_process_group()
    except Exception:
        queue.put((rank, "error", traceback.format_exc()))


def _run(scenario):
    ctx = mp.get_context("spawn")
    queue, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, scenario, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    return results


def test_shard_covers_the_batch_without_overlap():
    from grad_b200.replicas import shard

    for total in (100, 4096, 7, 1):
        for count in (1, 2, 4, 8):
            parts = [shard(total, count, i) for i in range(count)]
            assert parts[0][0] == 0 and parts[-1][1] == total
            assert all(parts[i][1] == parts[i + 1][0] for i in range(count - 1))


def test_two_ranks_meet_at_the_barrier_and_share_the_id():
    results = _run("barrier")
    assert [r[1] for r in results] == ["ok", "ok"], results
    assert results[0][2] == results[1][2] == b"id-from-rank-0"
    assert results[0][3] == (0, 50) and results[1][3] == (50, 100)
    assert results[0][4] == (0, 2048) and results[1][4] == (2048, 4096)


def test_a_failing_replica_releases_the_barrier():
    results = _run("stop")
    assert results == [(0, "released"), (1, "stopped-others")], results
