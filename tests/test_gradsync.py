"""Sharded gradient reduction (reduce-scatter over fsdp + all-reduce over the replicas of a shard) on
four gloo ranks laid out as fsdp 2 x sp 2, against the plain sum over all ranks."""
import os
import subprocess
import sys
import textwrap

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_SCRIPT = textwrap.dedent("""
    import sys, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    from ringattention_b200.parallel.mesh import DeviceMesh
    from ringattention_b200.parallel import gradsync
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mesh = DeviceMesh("1,2,1,2")
    f, me = mesh.size("fsdp"), mesh.index("fsdp")
    rep = mesh.replica_group("fsdp")
    S, T = 1000, 37                                   # shard length, replicated tail
    g = torch.Generator().manual_seed(100 + rank)
    mine = torch.randn(f * S + T, generator=g, dtype=torch.float64)
    every = [torch.randn(f * S + T, generator=torch.Generator().manual_seed(100 + r), dtype=torch.float64)
             for r in range(world)]
    want = torch.stack(every).sum(0)
    buf = mine.clone()
    gradsync.reduce_gradients(buf, S, f, me, mesh.axis("fsdp").group, rep, bucket=300)
    ok = torch.allclose(buf[me * S:(me + 1) * S], want[me * S:(me + 1) * S])
    ok &= torch.allclose(buf[f * S:], want[f * S:])
    own = (buf[me * S:(me + 1) * S] ** 2).sum().reshape(1)
    tail = (buf[f * S:] ** 2).sum().reshape(1)
    tot = gradsync.global_sumsq(own, tail, mesh.axis("fsdp").group)
    ok &= torch.allclose(tot, (want ** 2).sum().reshape(1))
    # f == 1: plain all-reduce
    buf = mine.clone()
    gradsync.reduce_gradients(buf, f * S, 1, 0, None, None, bucket=512)
    ok &= torch.allclose(buf, want)
    print("RANK", rank, "OK" if ok else "FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)
""")


def test_sharded_gradient_reduction_on_four_gloo_ranks(tmp_path):
    script = tmp_path / "gradsync.py"
    script.write_text(_SCRIPT.format(repo=REPO))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29627", str(script)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("OK") == 4
