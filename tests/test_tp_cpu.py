"""Tensor parallelism as two gloo ranks on the CPU: sharded weights, partial sums reduced with the norm, sharded arg-max,
the leader / follower step protocol — and a rank that leaves between steps (the survivor must get an error, not hang)."""
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(case, timeout=240, extra=()):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_tp_cpu_worker.py"), case, *extra]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    print(r.stdout[-2000:])
    print(r.stderr[-2000:])
    return r


def test_two_rank_generation_matches_one_rank():
    r = _run("generate")
    assert r.returncode == 0
    assert "tokens equal to the single-process run" in r.stdout


def test_rank_leaving_between_steps_fails_the_step_not_the_server():
    r = _run("rank_leaves")
    assert "peer left: request failed" in r.stdout


def test_mtp_drafter_under_two_tensor_parallel_ranks():
    r = _run("mtp")
    assert r.returncode == 0
    assert "MTP k=4 under TP 2" in r.stdout


def test_two_pipeline_stages_match_one_process():
    r = _run("pipeline")
    assert r.returncode == 0
    assert "two stages give the single-process tokens" in r.stdout


def test_expert_parallel_ranks_with_a_heat_aware_placement(tmp_path):
    r = _run("expert_placement", extra=(str(tmp_path / "heat.bin"),))
    assert r.returncode == 0
    assert "tokens equal to the single-process run" in r.stdout
