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


_ZERO_SCRIPT = textwrap.dedent("""
    import sys, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    from ringattention_b200.parallel.mesh import DeviceMesh
    from ringattention_b200.parallel import gradsync
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    def adamw(p, m, v, g, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip_coef=1.0):
        g = g * clip_coef
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        p.mul_(1 - lr * wd).addcdiv_(m / (1 - b1), (v / (1 - b2)).sqrt() + eps, value=-lr)

    ok = True
    for mesh_text in ("1,2,1,2", "1,1,1,4", "2,1,1,2"):
        mesh = DeviceMesh(mesh_text, register=False)
        f, me = mesh.size("fsdp"), mesh.index("fsdp")
        fg = mesh.axis("fsdp").group if f > 1 else None
        rep = mesh.replica_group("fsdp") if f > 1 else dist.group.WORLD
        zero = (dist.get_rank(rep), dist.get_world_size(rep), rep)
        S, T = 1024, 64                                  # shard region and tail (divisible by the slice count)
        gen = lambda r: torch.Generator().manual_seed(7 + r)
        grads = [torch.randn(f * S + T, generator=gen(r), dtype=torch.float64) for r in range(world)]
        total = torch.stack(grads).sum(0)
        w0 = torch.randn(f * S + T, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
        # --- replicated optimizer: every rank updates its whole shard region and the tail from the full sum
        want = w0.clone()
        gn = total.pow(2).sum().sqrt()
        coef = min(1.0, 1.0 / float(gn))
        adamw(want, torch.zeros_like(want), torch.zeros_like(want), total, clip_coef=coef)
        # --- sharded optimizer state
        g = grads[rank].clone()
        gradsync.reduce_gradients_zero(g, S, f, me, fg, zero)
        own_s = gradsync._slice(g[me * S:(me + 1) * S], zero[0], zero[1])
        own_t = gradsync._slice(g[f * S:], zero[0], zero[1])
        sq = gradsync.global_sumsq_zero(own_s.pow(2).sum().reshape(1), own_t.pow(2).sum().reshape(1), fg, zero)
        ok &= torch.allclose(sq, total.pow(2).sum().reshape(1))
        coef2 = min(1.0, 1.0 / float(sq.sqrt()))
        w = w0.clone()                                   # the "bf16 working copy": full shard region + tail
        for region, own_g in ((w[me * S:(me + 1) * S], own_s), (w[f * S:], own_t)):
            p = gradsync._slice(region, zero[0], zero[1])  # master slice aliases the working copy in this test
            adamw(p, torch.zeros_like(p), torch.zeros_like(p), own_g, clip_coef=coef2)
            gradsync.all_gather_(region, zero[0], zero[1], zero[2])
        ok &= torch.allclose(w[me * S:(me + 1) * S], want[me * S:(me + 1) * S])
        ok &= torch.allclose(w[f * S:], want[f * S:])
    print("RANK", rank, "OK" if ok else "FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)
""")


def test_optimizer_state_sharded_over_replicas_matches_replicated(tmp_path):
    """Reduce-scatter + AdamW on the owned slice + all-gather gives the weights of the replicated optimizer, on
    fsdp 2 x sp 2, sp 4 and dp 2 x sp 2 (four gloo ranks)."""
    script = tmp_path / "zero.py"
    script.write_text(_ZERO_SCRIPT.format(repo=REPO))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29628", str(script)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("OK") == 4
