"""Failure handling of the gradient-mean communicator, driven from the host without a GPU.

The reference releases the replicas that wait on a failed one (`Replicas.stop`, src/nn/replicas.zig:36-53;
tests/replicas.zig:105-118).  A device collective cannot be released that way, so `gb_comm_*` bounds every wait
with a host deadline and aborts the communicator when it passes.  Here the failing NCCL calls are faked
(tests/fake_nccl.c, loaded through GB_NCCL_LIBRARY): a communicator that never becomes ready, an allreduce whose
peer never joins, an asynchronous error.  Each scenario runs in a child process because the library binds NCCL
once per process.  The last test is the barrier-before-the-mean rule with two gloo ranks: a replica that fails
between steps releases the other with `Stopped` before it has enqueued anything.
"""
import multiprocessing as mp
import os
import socket
import subprocess
import sys
import textwrap
import traceback

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), os.path.join(HERE, "fake_nccl.c")], check=True)
    return str(out)


def _child(fake_lib, tmp_path, mode, body, timeout_ms=200):
    log = tmp_path / f"{mode}.log"
    env = dict(os.environ, GB_NCCL_LIBRARY=fake_lib, FAKE_NCCL_MODE=mode, FAKE_NCCL_LOG=str(log), GB_COMM_TIMEOUT_MS=str(timeout_ms),
               PYTHONPATH=ROOT)
    script = textwrap.dedent("""
        import ctypes as C, time
        from grad_b200 import abi
        lib = abi.library()
        ident = (C.c_ubyte * 128)()
        assert lib.gb_comm_unique_id(ident) == 0
        comm = C.c_void_p()
        t0 = time.monotonic()
        rc_create = lib.gb_comm_create(2, 0, ident, -1, C.byref(comm))
        buf = (C.c_float * 16)()
    """) + textwrap.dedent(body)
    res = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=120)
    calls = log.read_text().splitlines() if log.exists() else []
    return res, calls


def test_allreduce_is_one_ncclavg_call_on_the_flat_vector(fake_lib, tmp_path):
    res, calls = _child(fake_lib, tmp_path, "ok", """
        assert rc_create == 0
        assert lib.gb_allreduce_mean(comm, None, buf, 16) == 0
        lib.gb_comm_destroy(comm)
        print("done")
    """)
    assert res.returncode == 0 and "done" in res.stdout, res.stderr
    assert "ncclAllReduce count=16 dtype=7 op=4" in calls          # ncclFloat32, ncclAvg: no separate scale pass
    assert calls[-1] == "ncclCommDestroy" and "ncclCommAbort" not in calls


def test_a_communicator_that_never_becomes_ready_times_out(fake_lib, tmp_path):
    res, calls = _child(fake_lib, tmp_path, "hang_init", """
        waited = time.monotonic() - t0
        assert rc_create == 5, rc_create            # GB_ERR_TIMEOUT
        assert 0.15 <= waited < 20, waited
        assert not comm.value
        print("done")
    """)
    assert res.returncode == 0 and "done" in res.stdout, res.stderr
    assert "ncclCommAbort" in calls


def test_an_allreduce_whose_peer_never_joins_aborts_after_the_deadline(fake_lib, tmp_path):
    res, calls = _child(fake_lib, tmp_path, "hang_allreduce", """
        assert rc_create == 0
        assert lib.gb_comm_set_timeout(comm, 300) == 0
        t1 = time.monotonic()
        rc = lib.gb_allreduce_mean(comm, None, buf, 16)
        waited = time.monotonic() - t1
        assert rc == 5, rc                          # GB_ERR_TIMEOUT, not an endless wait
        assert 0.25 <= waited < 20, waited
        assert lib.gb_allreduce_mean(comm, None, buf, 16) == 6    # GB_ERR_NCCL: the communicator is gone (error.Stopped)
        assert lib.gb_comm_finish(comm, None) == 6
        lib.gb_comm_destroy(comm)
        print("done")
    """)
    assert res.returncode == 0 and "done" in res.stdout, res.stderr
    assert calls.count("ncclCommAbort") == 1
    assert sum(c.startswith("ncclAllReduce") for c in calls) == 1     # the second call never reached NCCL


def test_an_asynchronous_nccl_error_aborts_the_communicator(fake_lib, tmp_path):
    res, calls = _child(fake_lib, tmp_path, "error", """
        assert rc_create == 0
        assert lib.gb_allreduce_mean(comm, None, buf, 16) == 6      # GB_ERR_NCCL
        lib.gb_comm_destroy(comm)
        print("done")
    """)
    assert res.returncode == 0 and "done" in res.stdout, res.stderr
    assert "ncclCommAbort" in calls


# ---- barrier before the mean: two gloo ranks, fake NCCL, no GPU ------------------------------------------------
def _rank(rank, world, port, fake_lib, log_dir, queue):
    try:
        log = os.path.join(log_dir, f"rank{rank}.log")
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), GB_NCCL_LIBRARY=fake_lib,
                          FAKE_NCCL_MODE="ok", FAKE_NCCL_LOG=log)
        import torch
        import torch.distributed as dist

        from grad_b200.replicas import Replicas, Stopped, flat_grads

        dist.init_process_group("gloo", rank=rank, world_size=world)
        group = Replicas(world, rank, device=-1, timeout_s=20)
        flat, views = flat_grads([(8, 4), (5,), (3, 3)], "cpu")
        group.averageGrads(views)                       # step 1: every replica is alive
        if rank == 1:
            group.stop()                                # this replica fails between steps
            outcome = "stopped"
        else:
            try:
                group.averageGrads(views)               # step 2 must not enqueue a collective nobody will join
                outcome = "not released"
            except Stopped:
                outcome = "released"
        calls = open(log).read().splitlines()
        queue.put((rank, outcome, sum(c.startswith("ncclAllReduce") for c in calls), [c for c in calls if c.startswith("ncclAllReduce")][:1],
                   "ncclCommAbort" in calls, int(flat.numel())))
        group.close()
        dist.destroy_process_group()
    except Exception:
        queue.put((rank, "error", traceback.format_exc()))


def test_a_replica_that_fails_between_steps_releases_the_other_before_the_mean(fake_lib, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, fake_lib, str(tmp_path), queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in results] == ["released", "stopped"], results
    # views of one flat buffer went out as ONE call over the whole span (8*4 + pad 0 + 5 + pad 3 + 9 = 49 floats)
    assert results[0][2] == 1 and results[0][3] == ["ncclAllReduce count=49 dtype=7 op=4"], results
    assert results[0][4] and results[1][4]              # both aborted their communicators
    assert results[0][5] == 49
