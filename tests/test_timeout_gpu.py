"""The bounded device-side waits, made to run out on the host's request.

Every mbarrier wait in the contraction kernels gives up after a limit of polls, raises a CTA-wide abort flag, and the
kernel returns by itself with a status word that `gb_last_status` reports as GB_ERR_TIMEOUT -- the device-side
counterpart of a failed replica releasing the others (src/nn/replicas.zig:36-53).  Nothing here faults, traps or
hangs the GPU: the environment asks the library to leave out the copies of ONE K block of the first launch (a "stage
full" flag that nothing sets) and to shorten the poll limit, the consumer's wait runs out after a fraction of a
millisecond, every role leaves its loop, and the next ordinary product on the same handle must be correct.  The
knobs are read once per process, hence the child process.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_a_wait_that_runs_out_reports_timeout_and_leaves_the_handle_usable():
    script = textwrap.dedent("""
        import numpy as np, torch
        import grad_b200
        from grad_b200 import GbError, MatmulOpts, MatmulShape
        from oracle import binding as orc

        gpu = grad_b200.Gpu(0)
        m, n, k = 128, 64, 1024                      # one single-CTA tile, sixteen K blocks
        rng = np.random.default_rng(3)
        a = orc.bf16_round(rng.standard_normal((m, k), dtype=np.float32))
        b = orc.bf16_round(rng.standard_normal((k, n), dtype=np.float32))
        da, db = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()
        out = torch.zeros((m, n), device="cuda")
        gpu.matmul(da, db, out, MatmulShape(m, n, k), MatmulOpts())      # K block 3 of this launch is never copied
        plan = gpu.last_plan()
        assert plan["tensor_path"] == 1 and plan["tile_m"] == 128 and plan["splits"] == 1, plan
        try:
            gpu.check_status()
            raise SystemExit("the wait did not run out")
        except GbError as e:
            assert e.status == 5, e                  # GB_ERR_TIMEOUT
        assert gpu.check_status() == 0               # the status word was cleared by the read
        gpu.matmul(da, db, out, MatmulShape(m, n, k), MatmulOpts())      # the injection covered one launch only
        torch.cuda.synchronize()
        assert gpu.check_status() == 0
        want = orc.matmul_tiled(a, b, m, k, n, threads=orc.host_threads())
        err = float(np.linalg.norm(out.cpu().numpy() - want) / np.linalg.norm(want))
        assert err <= 2e-2, err
        gpu.close()
        print("timeout path ok", err)
    """)
    env = dict(os.environ, PYTHONPATH=ROOT, GB_TEST_SPIN_LIMIT="4000", GB_TEST_DROP_KBLOCK="3", GB_TEST_DROP_CALLS="1")
    res = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "timeout path ok" in res.stdout, res.stdout + res.stderr
