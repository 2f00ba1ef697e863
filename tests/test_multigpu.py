"""Multi-GPU tests (2 GPUs): in-kernel all-reduce over peer memory / NVSwitch multimem, the fused
all-reduce + residual + RMSNorm (+ quantise) kernel, and tensor-parallel decoding through the fused path."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _run(case, multicast="1", nproc=2, fusion=None):
    env = dict(os.environ, BLAZE_TEST_MULTICAST=multicast, NCCL_DEBUG="WARN")
    if fusion:
        env["BLAZE_TP_FUSION"] = fusion
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "_tp_worker.py"), case]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:])
    print(r.stderr[-3000:])
    assert r.returncode == 0


@pytest.mark.parametrize("multicast", ["1", "0"])
def test_allreduce(multicast):
    _run("allreduce", multicast)


@pytest.mark.parametrize("multicast", ["1", "0"])
def test_reduce_norm(multicast):
    _run("reduce_norm", multicast)


def test_gemm_allreduce_one_kernel():
    _run("gemm_allreduce")


@pytest.mark.parametrize("multicast", ["1", "0"])
def test_gemm_push_reduce_scatter(multicast):
    """Row-cut GEMM whose epilogue pushes the partial rows to their owner ranks + the owner's flag-started reduce / norm."""
    _run("push_reduce_norm", multicast)


@pytest.mark.parametrize("fusion", ["gemm_red", "reduce_norm", "rs_push"])
def test_tp2_model_fused_matches_tp1(fusion):
    _run("model", fusion=fusion)


def test_two_pipeline_stages_over_nccl():
    """Layers split over two GPUs, hidden rows handed over with isend / irecv in micro-batches, tokens returned to rank 0."""
    _run("pipeline")
