"""Tensor parallelism on two B200s against the unsharded CPU oracle: the sum over ranks after o_proj and down_proj
(the library's peer-memory exchange kernel by default, NCCL as the alternative) and the greedy merge over vocabulary
blocks.  Skipped on a one-GPU box.  NVLS is switched off: the ranks are child processes and nothing here needs
in-switch reduction."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
two_gpus = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


def run_ranks(worker: str, world: int = 2, limit: float = 240.0, **extra_env) -> list[str]:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    path = os.path.join(os.path.dirname(__file__), worker)
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", **extra_env)
        procs.append(subprocess.Popen([sys.executable, path], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=limit)[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-2000:] for o in outs)
    return outs


@two_gpus
@pytest.mark.parametrize("reduce", ["peer1", "peer2", "nccl"])
def test_two_gpu_tensor_parallel_decoder_matches_the_oracle(reduce):
    outs = run_ranks("tp_worker.py", TLALOC_B200_TP_REDUCE=reduce)
    assert "TP2 ok" in outs[0]


@two_gpus
@pytest.mark.parametrize("reduce", ["peer1", "peer2"])
def test_two_gpu_decoder_on_the_int8_tensor_core_form_matches_the_oracle(reduce):
    """Batch 32: the layers' projections on the int8 form; with the two-phase sum the residual stream is distributed by
    rows and the exchange hands the next projection its int8 planes."""
    outs = run_ranks("tp_worker.py", limit=400.0, TLALOC_B200_TP_REDUCE=reduce, TP_WORKER_BATCH="32")
    assert "TP2 ok" in outs[0]


@two_gpus
def test_peer_memory_sum_is_exact_and_identical_on_both_ranks():
    outs = run_ranks("peer_worker.py")
    assert "peer sum ok" in outs[0]
