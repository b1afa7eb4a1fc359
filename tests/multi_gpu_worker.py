"""Worker run under torchrun by test_gpu_multi.py: one process per visible GPU (2, 4 or 8), NVLS off.

Every check compares against a one-device computation of the same thing (the dense fp32 oracle for the ops, a
stand-alone single-device trainer for the model) and judges gradients by their largest error relative to the
largest reference entry, tensor by tensor."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ringattention_b200 as rab  # noqa: E402
from ringattention_b200 import ringattention  # noqa: E402
from ringattention_b200.config import LlamaConfig, TrainConfig  # noqa: E402
from ringattention_b200.ops import _lib, reference as R  # noqa: E402
from ringattention_b200.parallel.mesh import DeviceMesh  # noqa: E402
from ringattention_b200.trainer import PeerLost, Trainer, init_distributed  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


def bcast(*ts):
    for t in ts:
        dist.broadcast(t, 0)


# ------------------------------------------------------------------------------------------------ ops
def ring_vs_dense(rank, world, dev):
    """``ringattention`` over the whole ring, both layouts, causal and packed documents, against dense fp32."""
    ok = True
    B, H, D, Sl = 1, 4, 128, 512
    S = Sl * world
    for layout in ("contiguous", "zigzag"):
        for cbs, seg in ((1, False), (None, True), (1, True)):
            torch.manual_seed(0)
            q, k, v, do = [torch.randn(B, S, H, D, device=dev).bfloat16() for _ in range(4)]
            bcast(q, k, v, do)
            ids = None
            if seg:
                ids = torch.cumsum((torch.rand(B, S, device=dev) < 0.004).int(), 1).int()
                bcast(ids)
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
            g = max(rel(ql.grad, qf.grad.index_select(1, pos)), rel(kl.grad, kf.grad.index_select(1, pos)),
                    rel(vl.grad, vf.grad.index_select(1, pos)))
            ok &= e < 0.03 and g < 0.03
            print(f"[{rank}] ring {layout} cbs={cbs} seg={seg}: out {e:.4f} grad {g:.4f}", flush=True)
    return ok


def cache_idx_and_inference_op(rank, world, dev):
    """Replicated queries against the sequence-sharded cache: ``ringattention(..., cache_idx=...)`` (causal) and
    ``ringattention_inference`` (boolean mask) for query lengths on both sides of the decode kernel, with
    gradients: dK/dV of the local shard, dQ complete on every rank."""
    ok = True
    B, H, D, Sl = 2, 2, 128, 640
    S = Sl * world
    sl = slice(rank * Sl, (rank + 1) * Sl)
    for ql in (1, 8, 100, 2048):
        torch.manual_seed(ql)
        q = torch.randn(B, ql, H, D, device=dev).bfloat16()
        k, v = torch.randn(B, S, H, D, device=dev).bfloat16(), torch.randn(B, S, H, D, device=dev).bfloat16()
        do = torch.randn(B, ql, H, D, device=dev).bfloat16()
        mask = (torch.rand(B, 1, ql, S, device=dev) < 0.6).to(torch.uint8)
        mask[..., 0] = 1
        bcast(q, k, v, do, mask)
        mask = mask.bool()
        qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
        ref = R.dense_attention(qf, kf, vf, extra_masked=~mask, dtype=torch.float32)
        ref.backward(do.float())
        for _ in range(2):  # twice: the inbox is double-buffered across calls
            ql_, kl, vl = [t.clone().requires_grad_(True) for t in (q, k[:, sl].contiguous(), v[:, sl].contiguous())]
            out = rab.ringattention_inference(ql_, kl, vl, mask, "sp")
            out.backward(do)
        with torch.no_grad():
            out_ng = rab.ringattention_inference(q, k[:, sl].contiguous(), v[:, sl].contiguous(), mask, "sp")
        torch.cuda.synchronize()
        _lib.check_status()
        e = max((out.float() - ref).abs().max().item(), (out_ng.float() - ref).abs().max().item())
        g = max(rel(ql_.grad, qf.grad), rel(kl.grad, kf.grad[:, sl]), rel(vl.grad, vf.grad[:, sl]))
        ok &= e < 0.02 and g < 0.03
        print(f"[{rank}] inference op q_len={ql}: out {e:.4f} grad {g:.4f}", flush=True)
    # cache_idx: queries at positions cache_idx.. on every rank, causal against the sharded cache
    for ql, cache_idx in ((128, S - 256), (100, S - 229)):
        torch.manual_seed(cache_idx)
        q = torch.randn(B, ql, H, D, device=dev).bfloat16()
        k, v = torch.randn(B, S, H, D, device=dev).bfloat16(), torch.randn(B, S, H, D, device=dev).bfloat16()
        bcast(q, k, v)
        kw = dict(causal_block_size=1, query_chunk_size=128, key_chunk_size=128)
        out = ringattention(q, k[:, sl].contiguous(), v[:, sl].contiguous(), None, None, cache_idx, "sp", True, kw)
        ref = R.dense_attention(q, k, v, torch.arange(cache_idx, cache_idx + ql, device=dev),
                                torch.arange(S, device=dev), causal_block_size=1, dtype=torch.float32)
        torch.cuda.synchronize()
        _lib.check_status()
        e = (out.float() - ref).abs().max().item()
        ok &= e < 0.02
        print(f"[{rank}] cache_idx={cache_idx} q_len={ql}: out {e:.4f}", flush=True)
    return ok


def decode_engine(rank, world, dev):
    """The inference engine on a sharded cache against the same engine on one device."""
    from ringattention_b200.models.llama_infer import LlamaInference

    ok = True
    cfg = LlamaConfig.named("llama-tiny")
    chunk = 128 * world
    inf = LlamaInference(cfg, max_context=8 * chunk, batch=1, seed=5, axis="sp")
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (1, 2 * chunk), device=dev)
    bcast(prompt)
    logits = None
    for c0 in range(0, prompt.shape[1], chunk):
        logits = inf.prefill_chunk(prompt[:, c0:c0 + chunk])
    single = LlamaInference(cfg, max_context=8 * chunk, batch=1, seed=5, axis=None)
    logits1 = None
    for c0 in range(0, prompt.shape[1], chunk):
        logits1 = single.prefill_chunk(prompt[:, c0:c0 + chunk])
    e = rel(logits, logits1)
    ok &= e < 0.03
    print(f"[{rank}] prefill logits on the sharded cache vs one device: rel {e:.4f}", flush=True)
    # teacher-forced decode: feed both engines the same tokens and compare the logits of every step
    tok = logits1.argmax(dim=-1)
    worst = 0.0
    for _ in range(6):
        la, lb = inf.decode_step(tok), single.decode_step(tok)
        worst = max(worst, rel(la, lb))
        tok = lb.argmax(dim=-1)
    ok &= worst < 0.03
    print(f"[{rank}] decode logits, 6 teacher-forced steps: worst rel {worst:.4f}", flush=True)
    # the same steps replayed from a CUDA graph (every exchange of the step inside the graph): the graph must give
    # the logits of the eager step from the same state, which the single-device engine provides
    agree = 0
    for _ in range(4):
        inf._tok_buf.copy_(tok.to(torch.int32).reshape(-1))
        lb = single.decode_step(tok)
        ta = inf.decode_step_graph().clone()
        top2 = lb.topk(2).values[0]
        # the graph's greedy token is the single-device argmax unless the two best logits are within bf16 noise
        agree += int(ta[0]) == int(lb.argmax(dim=-1)[0]) or float(top2[0] - top2[1]) < 0.05 * float(lb.abs().max())
        tok = lb.argmax(dim=-1)
    ok &= agree == 4
    print(f"[{rank}] graph-replayed sharded decode: {agree}/4 greedy tokens agree with one device", flush=True)
    # three streams on one shared context (striped over the ring), private tails dealt round-robin to the ranks
    sh = LlamaInference(cfg, max_context=8 * chunk, batch=1, seed=5, axis="sp", streams=3, max_new_tokens=16)
    sh1 = LlamaInference(cfg, max_context=8 * chunk, batch=1, seed=5, axis=None, streams=3, max_new_tokens=16)
    for c0 in range(0, prompt.shape[1], chunk):
        la, lb = sh.prefill_chunk(prompt[:, c0:c0 + chunk]), sh1.prefill_chunk(prompt[:, c0:c0 + chunk])
    tok = lb[0].topk(3).indices
    worst = 0.0
    for _ in range(2 * world + 1):
        la, lb = sh.decode_step(tok), sh1.decode_step(tok)
        worst = max(worst, rel(la, lb))
        tok = lb.argmax(dim=-1)
    ok &= worst < 0.03
    print(f"[{rank}] shared-prefix decode, 3 streams: worst rel {worst:.4f}", flush=True)
    torch.cuda.synchronize()
    _lib.check_status()
    return ok


# ------------------------------------------------------------------------------------------------ model
def _reference_gradients(cfg_name, seed, tokens, targets, seg, dev):
    """Gradients and loss of the whole global batch on one device (a stand-alone trainer: joins no collective)."""
    cfg = LlamaConfig.named(cfg_name)
    tc = TrainConfig(model=cfg_name, mesh="1,1,1,1", seq_len=tokens.shape[1], global_batch=tokens.shape[0],
                     lr=1e-3, seed=seed)
    ref = Trainer(cfg, tc, standalone=True)
    P = ref.model.params
    P.ensure_grads().zero_()
    loss = ref.model.forward_backward(tokens.to(dev), targets.to(dev), ref.context(seg))
    return ref, P, float(loss) / (tokens.shape[0] * tokens.shape[1])


def _grad_errors(tr, P_ref):
    """Largest relative error per parameter tensor of the reduced gradient this rank owns."""
    P = tr.model.params
    worst, worst_name = 0.0, ""
    for name in P.index:
        want = P_ref.g(name)
        if name in P.rep or P.shard_count == 1:
            got = P.g(name)
        else:  # fsdp: this rank holds the sum of its own rows only
            off, N, Kd, sr = P.mat[name]
            r0 = P.shard_index * sr
            rows = max(0, min(sr, N - r0))
            if rows == 0:
                continue
            got = P.grad_shard(P.shard_index)[off:off + rows * Kd].view(rows, Kd)
            want = want[r0:r0 + rows]
        e = rel(got, want)
        if e > worst:
            worst, worst_name = e, name
    return worst, worst_name


def mesh_parity(rank, world, dev, mesh_text, label, packed=0):
    """Gradients after the mesh-wide reduction, a 5-step loss curve, and (with the optimizer state sharded over
    the replicas, the default) the same 5-step curve again, against a single-device trainer on the same batches."""
    ok = True
    mesh = DeviceMesh(mesh_text, register=False)
    sp, batch_groups = mesh.size("sp"), mesh.size("dp") * mesh.size("fsdp")
    cfg = LlamaConfig.named("llama-tiny", layout="zigzag" if sp > 1 else "contiguous")
    seq, gb = 512 * sp, batch_groups
    curves = {}
    for zero1 in (False, True):
        tc = TrainConfig(model="llama-tiny", mesh=mesh_text, seq_len=seq, global_batch=gb, lr=1e-3, seed=11,
                         zero1=zero1, packed_mean_doc_len=packed)
        tr = Trainer(cfg, tc, mesh=DeviceMesh(mesh_text, register=False))
        tokens, targets, seg = tr.make_global_batch()
        if not zero1:
            # ---- gradients of one batch, reduced over the mesh, against one device
            ref, P_ref, loss_ref = _reference_gradients("llama-tiny", 11, tokens, targets, seg, dev)
            tok, tgt = tr.shard_batch(tokens, targets, seg)
            P = tr.model.params
            P.ensure_grads().zero_()
            loss_sum = tr.model.forward_backward(tok.to(dev).contiguous(), tgt.to(dev).contiguous(), tr.context(seg))
            dist.all_reduce(loss_sum)
            tr._all_reduce_grads()
            torch.cuda.synchronize()
            _lib.check_status()
            worst, name = _grad_errors(tr, P_ref)
            dl = abs(float(loss_sum) / (gb * seq) - loss_ref)
            ok &= worst < 0.02 and dl < 1e-3
            print(f"[{rank}] {label}: reduced gradients worst rel err {worst:.4f} ({name}), loss diff {dl:.5f}", flush=True)
            ref_losses = [ref.train_step(tokens, targets, seg) for _ in range(5)]
            curves["ref"] = ref_losses
        curves[zero1] = [tr.train_step(tokens, targets, seg) for _ in range(5)]
        d = max(abs(a - b) for a, b in zip(curves[zero1], curves["ref"]))
        ok &= d < 5e-3 and curves[zero1][-1] < curves[zero1][0]
        print(f"[{rank}] {label} zero1={zero1}: losses {[round(x, 4) for x in curves[zero1]]} vs one device "
              f"{[round(x, 4) for x in curves['ref']]} (max diff {d:.4f})", flush=True)
        last = tr
    torch.cuda.synchronize()
    _lib.check_status()
    return ok, last, (tokens, targets, seg)


def checkpoint_resume(rank, world, dev, tr, batch, label):
    """Save (sharded optimizer state, one file per rank), train on, reload into a fresh trainer on the same mesh,
    and get the same losses."""
    tokens, targets, seg = batch
    d = [tempfile.mkdtemp(prefix="ra_ckpt_") if rank == 0 else None]
    dist.broadcast_object_list(d, 0)
    tr.save_checkpoint(d[0])
    after = [tr.train_step(tokens, targets, seg) for _ in range(3)]
    tr2 = Trainer(tr.cfg, tr.tc, mesh=DeviceMesh(tr.tc.mesh, register=False))
    tr2.load_checkpoint(d[0])
    resumed = [tr2.train_step(tokens, targets, seg) for _ in range(3)]
    dmax = max(abs(a - b) for a, b in zip(after, resumed))
    print(f"[{rank}] {label}: checkpoint resume losses {resumed} vs {after}", flush=True)
    return dmax < 2e-3


def peer_loss(rank, world, dev):
    """A rank leaves between steps; the others learn of it on the host before they launch anything."""
    import time

    cfg = LlamaConfig.named("llama-tiny", layout="zigzag")
    tc = TrainConfig(model="llama-tiny", mesh=f"1,1,1,{world}", seq_len=512 * world, global_batch=1, lr=1e-3, seed=11)
    tr = Trainer(cfg, tc)
    tokens, targets, seg = tr.make_global_batch()
    tr.train_step(tokens, targets, seg)
    dist.barrier()
    if rank == world - 1:
        tr.leave()
        print(f"[{rank}] left", flush=True)
        return True
    time.sleep(1.0)
    ok = True
    try:
        tr.train_step(tokens, targets, seg)
        ok = False
        print(f"[{rank}] peer loss NOT detected", flush=True)
    except PeerLost as e:
        print(f"[{rank}] detected: {e}", flush=True)
    ok &= float((torch.ones(4, device=dev) * 3).sum()) == 12.0  # the context is still usable
    return ok


def main():
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    DeviceMesh(f"1,1,1,{world}")  # registers the "sp" axis for the op-level checks
    ok = ring_vs_dense(rank, world, dev)
    ok &= cache_idx_and_inference_op(rank, world, dev)
    ok &= decode_engine(rank, world, dev)
    ok1, _, _ = mesh_parity(rank, world, dev, f"1,1,1,{world}", f"sp={world}")
    ok &= ok1
    ok1, tr_f, batch_f = mesh_parity(rank, world, dev, f"1,2,1,{world // 2}", f"fsdp=2 x sp={world // 2}", packed=96)
    ok &= ok1
    ok &= checkpoint_resume(rank, world, dev, tr_f, batch_f, f"fsdp=2 x sp={world // 2}")
    ok1, _, _ = mesh_parity(rank, world, dev, f"2,1,1,{world // 2}", f"dp=2 x sp={world // 2}")
    ok &= ok1
    ok &= peer_loss(rank, world, dev)
    print(f"[{rank}] RESULT {'OK' if ok else 'FAIL'}", flush=True)
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
