"""Worker run under torchrun by test_gpu_multi.py (one process per GPU, NVLS off)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ringattention_b200 import ringattention  # noqa: E402
from ringattention_b200.config import LlamaConfig, TrainConfig  # noqa: E402
from ringattention_b200.ops import _lib, reference as R  # noqa: E402
from ringattention_b200.trainer import PeerLost, Trainer, init_distributed  # noqa: E402


def ring_vs_dense(rank, world, dev):
    ok = True
    B, H, D, Sl = 1, 4, 128, 512
    S = Sl * world
    for layout in ("contiguous", "zigzag"):
        for cbs, seg in ((1, False), (None, True)):
            torch.manual_seed(0)
            q, k, v, do = [torch.randn(B, S, H, D, device=dev).bfloat16() for _ in range(4)]
            for t in (q, k, v, do):
                dist.broadcast(t, 0)
            ids = None
            if seg:
                ids = torch.cumsum((torch.rand(B, S, device=dev) < 0.004).int(), 1).int()
                dist.broadcast(ids, 0)
            pos = R.shard_positions(rank, world, Sl, layout, dev)
            ql, kl, vl = [t.index_select(1, pos).contiguous().requires_grad_(True) for t in (q, k, v)]
            kw = dict(causal_block_size=cbs, query_chunk_size=128, key_chunk_size=128, layout=layout)
            out = ringattention(ql, kl, vl, None, ids, None, "sp", True, kw)
            out.backward(do.index_select(1, pos).contiguous())
            torch.cuda.synchronize()
            _lib.check_status()
            qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
            ref = R.dense_attention(qf, kf, vf, causal_block_size=cbs, seg_q=ids, seg_k=ids, dtype=torch.float32)
            ref.backward(do.float())
            e = (out.float() - ref.detach().index_select(1, pos)).abs().max().item()
            rel = lambda a, b: ((a.float() - b).abs().max() / (b.abs().max() + 1e-9)).item()
            g = max(rel(ql.grad, qf.grad.index_select(1, pos)), rel(kl.grad, kf.grad.index_select(1, pos)),
                    rel(vl.grad, vf.grad.index_select(1, pos)))
            ok &= e < 0.03 and g < 0.03
            print(f"[{rank}] ring {layout} cbs={cbs} seg={seg}: out {e:.4f} grad {g:.4f}", flush=True)
    return ok


def trainer_parity_and_peer_loss(rank, world, dev):
    cfg = LlamaConfig.named("llama-tiny", layout="zigzag")
    tc = TrainConfig(model="llama-tiny", mesh=f"1,1,1,{world}", seq_len=512 * world, global_batch=1, lr=1e-3, seed=11)
    tr = Trainer(cfg, tc)
    tokens, targets, seg = tr.make_global_batch()
    l_sp = tr.train_step(tokens, targets, seg)
    # same batch on one device (every rank computes it redundantly; only the loss is compared)
    from ringattention_b200.models.llama import LlamaModel
    ref_model = LlamaModel(LlamaConfig.named("llama-tiny"), dev, seed=11, with_optimizer=False)
    ctx = ref_model.make_context(1, 512 * world)
    l_ref = ref_model.forward_loss(tokens.to(dev), targets.to(dev), ctx).item() / (512 * world)
    ok = abs(l_sp - l_ref) < 2e-2
    print(f"[{rank}] trainer sp={world} loss {l_sp:.4f} vs single-device {l_ref:.4f}", flush=True)
    l2 = tr.train_step(tokens, targets, seg)
    ok &= l2 < l_sp
    # a rank leaves between steps; the others find out on the host before launching anything
    dist.barrier()
    if rank == world - 1:
        tr.leave()
        print(f"[{rank}] left", flush=True)
        return ok, True
    import time
    time.sleep(1.0)
    try:
        tr.train_step(tokens, targets, seg)
        ok = False
        print(f"[{rank}] peer loss NOT detected", flush=True)
    except PeerLost as e:
        print(f"[{rank}] detected: {e}", flush=True)
    ok &= float((torch.ones(4, device=dev) * 3).sum()) == 12.0  # context still usable
    return ok, False


def decode_and_inference(rank, world, dev):
    """Stationary-KV decode merged through peer stores, and the inference engine on a sharded cache,
    against one-device results."""
    import ringattention_b200 as rab
    from ringattention_b200.models.llama_infer import LlamaInference

    ok = True
    torch.manual_seed(1)
    B, QL, H, D, Sl = 2, 1, 4, 128, 640
    q = torch.randn(B, QL, H, D, device=dev).bfloat16()
    k = torch.randn(B, Sl * world, H, D, device=dev).bfloat16()
    v = torch.randn_like(k)
    mask = torch.rand(B, 1, QL, Sl * world, device=dev) < 0.8
    for t in (q, k, v):
        dist.broadcast(t, 0)
    mi = mask.to(torch.uint8)
    dist.broadcast(mi, 0)
    mask = mi.bool()
    sl = slice(rank * Sl, (rank + 1) * Sl)
    for _ in range(3):  # repeated calls exercise the double-buffered inbox
        out = rab.ringattention_inference(q, k[:, sl].contiguous(), v[:, sl].contiguous(), mask, "sp")
    ref = R.dense_attention(q, k, v, extra_masked=~mask, dtype=torch.float32)
    e = (out.float() - ref).abs().max().item()
    ok &= e < 0.02
    print(f"[{rank}] ring decode err {e:.4f}", flush=True)
    cfg = LlamaConfig.named("llama-tiny")
    inf = LlamaInference(cfg, max_context=2048, batch=1, seed=5, axis="sp")
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (1, 512), device=dev)
    dist.broadcast(prompt, 0)
    gen, _ = inf.generate(prompt, 6, chunk=256)
    single = LlamaInference(cfg, max_context=2048, batch=1, seed=5, axis=None)
    gen1, _ = single.generate(prompt, 6, chunk=256)
    agree = (gen == gen1).float().mean().item()
    ok &= agree >= 0.8
    print(f"[{rank}] sharded-cache generation agrees with one device on {agree:.2f} of tokens", flush=True)
    torch.cuda.synchronize()
    _lib.check_status()
    return ok


def fsdp_parity(rank, world, dev):
    """fsdp = world: weights row-sharded, remote shards gathered inside the GEMMs. The loss of the
    sharded run must equal a replicated single-device run on the same global batch, step after step."""
    from ringattention_b200.models.llama import LlamaModel
    from ringattention_b200.parallel.mesh import DeviceMesh

    ok = True
    cfg = LlamaConfig.named("llama-tiny")
    tc = TrainConfig(model="llama-tiny", mesh=f"1,{world},1,1", seq_len=512, global_batch=world, lr=1e-3, seed=21)
    tr = Trainer(cfg, tc, mesh=DeviceMesh(f"1,{world},1,1", register=False))
    tokens, targets, seg = tr.make_global_batch()
    # gather GEMMs against the assembled matrix
    P = tr.model.params
    name = "l0.wqkv"
    parts = [torch.zeros(P.mat[name][3], P.mat[name][2], device=dev, dtype=torch.bfloat16) for _ in range(world)]
    mine = torch.zeros_like(parts[0])
    ws = P.w_shard(name)
    mine[:ws.shape[0]] = ws
    dist.all_gather(parts, mine, group=tr.mesh.axis("fsdp").group)
    W = torch.cat(parts, 0)[:P.mat[name][1]]
    x = torch.randn(300, W.shape[1], device=dev).bfloat16()
    dy = torch.randn(300, W.shape[0], device=dev).bfloat16()
    y = P.lin_fwd(x, name)
    dx = P.lin_dgrad(dy, name)
    e1 = ((y.float() - x.float() @ W.float().t()).abs().max() / (x.float() @ W.float().t()).abs().max()).item()
    e2 = ((dx.float() - dy.float() @ W.float()).abs().max() / (dy.float() @ W.float()).abs().max()).item()
    ok &= e1 < 0.02 and e2 < 0.02
    print(f"[{rank}] gather GEMM fwd rel err {e1:.4f} dgrad rel err {e2:.4f}", flush=True)
    losses = [tr.train_step(tokens, targets, seg) for _ in range(3)]
    # replicated reference on one device (every rank computes it; only losses are compared)
    ref_tc = TrainConfig(model="llama-tiny", mesh="1,1,1,1", seq_len=512, global_batch=world, lr=1e-3, seed=21)
    ref = Trainer(cfg, ref_tc, standalone=True)
    ref_losses = [ref.train_step(tokens, targets, seg) for _ in range(3)]
    d = max(abs(a - b) for a, b in zip(losses, ref_losses))
    ok &= d < 3e-2 and losses[-1] < losses[0]
    print(f"[{rank}] fsdp losses {[round(v, 4) for v in losses]} vs replicated {[round(v, 4) for v in ref_losses]}", flush=True)
    torch.cuda.synchronize()
    _lib.check_status()
    return ok


def main():
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    from ringattention_b200.parallel.mesh import DeviceMesh

    DeviceMesh(f"1,1,1,{world}")
    ok = ring_vs_dense(rank, world, dev)
    ok &= decode_and_inference(rank, world, dev)
    ok &= fsdp_parity(rank, world, dev)
    ok2, left = trainer_parity_and_peer_loss(rank, world, dev)
    print(f"[{rank}] RESULT {'OK' if (ok and ok2) else 'FAIL'}", flush=True)
    os._exit(0 if (ok and ok2) else 1)


if __name__ == "__main__":
    main()
