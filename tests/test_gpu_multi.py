"""Multi-GPU tier on every GPU of the box (2, 4 or 8): the fused ring (KV pulled from peer memory inside the
kernels, dK/dV reduced into the owner's accumulators) against dense attention in both layouts, the inference op
and ``cache_idx`` on a sharded cache, gradient and loss-curve parity of the sp, fsdp x sp and dp x sp meshes
with a single-device trainer, checkpoint resume with sharded optimizer state, and host-side peer-loss
detection. Runs child processes under torchrun with NVLS disabled and a 5 s barrier timeout."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def test_ring_meshes_and_peer_loss_on_all_gpus():
    import torch

    n = torch.cuda.device_count()
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               RINGATTN_B200_BARRIER_TIMEOUT_S="5")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29641",
                        os.path.join(HERE, "multi_gpu_worker.py")],
                       capture_output=True, text=True, timeout=900, env=env)
    log = os.environ.get("RINGATTN_B200_MULTI_LOG")
    if log:
        with open(log, "w") as f:
            f.write(p.stdout + "\n---- stderr ----\n" + p.stderr[-20000:])
    tail = p.stdout[-6000:] + p.stderr[-3000:]
    assert p.stdout.count("RESULT OK") == n, tail
    assert "detected:" in p.stdout, tail
