"""Two-GPU tests of the fused ring (KV pulled from peer memory inside the kernels, dK/dV reduced
into the owner's accumulators), sequence-parallel training parity and host-side peer-loss
detection. Runs child processes under torchrun with NVLS disabled."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def test_two_gpu_ring_training_and_peer_loss():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               RINGATTN_B200_BARRIER_TIMEOUT_S="20")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29641",
                        os.path.join(HERE, "multi_gpu_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    tail = p.stdout[-3000:] + p.stderr[-3000:]
    assert p.stdout.count("RESULT OK") == 2, tail
    assert "detected:" in p.stdout, tail
