"""The N > 1 path of the benchmark on CPU: two gloo ranks, barrier + max-over-ranks timing + summed units."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, %r)
    import torch.distributed as dist
    from ittai_b200 import replicas
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    replicas.barrier()
    t0 = time.perf_counter()
    time.sleep(0.05 * (rank + 1))                  # rank 1 is the slow replica
    ms = (time.perf_counter() - t0) * 1e3
    replicas.barrier()
    (t_max, t_other), units = replicas.aggregate([ms, 10.0 * (rank + 1)], units=256 * (rank + 1))
    assert units == 256 * 3, units
    assert t_max >= 99.0 and t_other == 20.0, (t_max, t_other)
    if rank == 0:
        print("OK", round(t_max), units)
    dist.destroy_process_group()
""") % ROOT


def test_two_rank_aggregation_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env={**os.environ, "OMP_NUM_THREADS": "1"})
    assert r.returncode == 0, r.stdout + r.stderr
    assert "OK" in r.stdout


def test_single_process_aggregate_is_identity():
    from ittai_b200 import replicas
    (a, b), u = replicas.aggregate([1.5, 2.5], units=7)
    assert (a, b, u) == (1.5, 2.5, 7.0)
