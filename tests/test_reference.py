"""CPU tests of the PyTorch restatement: blockwise math, ring layer, masks, layouts."""
import math

import pytest
import torch

from ringattention_b200.config import BlockwiseKwargs
from ringattention_b200.ops import reference as R
from ringattention_b200.parallel.comm import SingleComm, run_fake_ring


def _rand(B, S, H, D, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, S, H, D, generator=g, dtype=dtype) for _ in range(3)]


@pytest.mark.parametrize("cbs", [None, 1, 4, 64])
@pytest.mark.parametrize("qc,kc", [(16, 16), (32, 8), (64, 64)])
def test_blockwise_matches_dense(cbs, qc, kc):
    q, k, v = _rand(2, 64, 3, 8)
    kw = BlockwiseKwargs(causal_block_size=cbs, query_chunk_size=qc, key_chunk_size=kc)
    pos = torch.arange(64)
    carry = R.new_carry(2, 64, 3, 8, "cpu", torch.float64)
    carry = R.blockwise_fwd(q, k, v, carry, pos, pos, kw, acc_dtype=torch.float64)
    out, lse = R.finalize(carry, torch.float64)
    ref, ref_lse = R.dense_attention(q, k, v, causal_block_size=cbs, return_lse=True)
    assert torch.allclose(out, ref, atol=1e-10)
    assert torch.allclose(lse, ref_lse, atol=1e-10)


def test_tile_visible_matches_bruteforce():
    for qc in (1, 2, 3, 8):
        for kc in (1, 2, 5, 8):
            for cbs in (1, 2, 4, 16):
                for q0 in range(0, 24, qc):
                    for k0 in range(0, 24, kc):
                        qp = torch.arange(q0, q0 + qc)
                        kp = torch.arange(k0, k0 + kc)
                        brute = bool(((qp[:, None] // cbs) >= (kp[None, :] // cbs)).any())
                        assert R.tile_visible(qp, kp, cbs) == brute


def test_blockwise_bwd_matches_autograd():
    q, k, v = _rand(1, 48, 2, 8, seed=1)
    g = torch.randn(1, 48, 2, 8, dtype=torch.float64)
    kw = BlockwiseKwargs(causal_block_size=1, query_chunk_size=16, key_chunk_size=12)
    pos = torch.arange(48)
    qa, ka, va = [t.clone().requires_grad_(True) for t in (q, k, v)]
    ref, lse = R.dense_attention(qa, ka, va, causal_block_size=1, return_lse=True)
    ref.backward(g)
    dq, dk, dv = R.blockwise_bwd(q, k, v, ref.detach(), lse.detach(), g, pos, pos, kw,
                                 acc_dtype=torch.float64)
    for a, b in ((dq, qa.grad), (dk, ka.grad), (dv, va.grad)):
        assert torch.allclose(a, b, atol=1e-9)


def _ring_case(world, layout, cbs, seg=False, bias=False, pdrop=0.0, dtype=torch.float32, S=2048,
               B=1, H=8, D=64, qc=256):
    g = torch.Generator().manual_seed(3)
    q, k, v, do = [torch.randn(B, S, H, D, generator=g, dtype=dtype) for _ in range(4)]
    ids = torch.zeros(B, S, dtype=torch.int32)
    if seg:
        ids = torch.cumsum((torch.rand(B, S, generator=g) < 0.01).int(), 1).int()
    bias_t = torch.zeros(B, 1, 1, S, dtype=dtype)
    if bias:
        bias_t = torch.randn(B, 1, 1, S, generator=g, dtype=dtype)
    kw = dict(causal_block_size=cbs, query_chunk_size=qc, key_chunk_size=qc, deterministic=pdrop == 0.0,
              dropout_rng=1234, attn_pdrop=pdrop, dtype=dtype, policy="nothing_saveable", precision=None,
              prevent_cse=True, layout=layout)
    Sl = S // world

    def body(comm):
        pos = R.shard_positions(comm.rank, world, Sl, layout)
        ql, kl, vl = [t.index_select(1, pos).clone().requires_grad_(True) for t in (q, k, v)]
        out = R.ring_attention_ref(ql, kl, vl, bias_t, ids, None, comm, True, kw)
        (out * do.index_select(1, pos)).sum().backward()
        return pos, out.detach(), ql.grad, kl.grad, vl.grad

    res = run_fake_ring(world, body)
    qa, ka, va = [t.double().requires_grad_(True) for t in (q, k, v)]
    seed = BlockwiseKwargs.from_any(kw).seed()
    ref = R.dense_attention(qa, ka, va, causal_block_size=cbs, bias=bias_t.double(), seg_q=ids, seg_k=ids,
                            seed=seed, pdrop=pdrop)
    (ref * do.double()).sum().backward()
    tol = 2e-4 if dtype == torch.float32 else 1e-9
    for pos, out, dq, dk, dv in res:
        assert torch.allclose(out.double(), ref.detach().index_select(1, pos), atol=tol)
        assert torch.allclose(dq.double(), qa.grad.index_select(1, pos), atol=tol * 5)
        assert torch.allclose(dk.double(), ka.grad.index_select(1, pos), atol=tol * 5)
        assert torch.allclose(dv.double(), va.grad.index_select(1, pos), atol=tol * 5)


def test_cpu_plumbing_config_four_rank_sp_mesh():
    """Batch 1, total seq 2048 (512 per rank), 8 heads of 64, fp32, causal, chunks 256, zero bias,
    zero segment ids, gradients from sum(out * g), against a dense causal softmax."""
    _ring_case(4, "contiguous", 1)


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("cbs", [None, 1, 128])
def test_ring_layouts_and_causality(layout, cbs):
    _ring_case(4, layout, cbs, S=512, H=2, D=16, qc=64, dtype=torch.float64)


def test_ring_segments_bias_dropout():
    _ring_case(2, "contiguous", 1, seg=True, bias=True, pdrop=0.1, S=256, H=2, D=16, qc=32,
               dtype=torch.float64)
    _ring_case(4, "zigzag", 1, seg=True, S=256, H=2, D=16, qc=32, dtype=torch.float64)


def test_dropout_statistics_and_determinism():
    qp, kp = torch.arange(512), torch.arange(512)
    d1 = R.dropped(99, 0.25, 2, 4, qp, kp)
    d2 = R.dropped(99, 0.25, 2, 4, qp, kp)
    d3 = R.dropped(100, 0.25, 2, 4, qp, kp)
    assert torch.equal(d1, d2)
    assert not torch.equal(d1, d3)
    assert abs(d1.float().mean().item() - 0.25) < 0.005
    # the mask of a shard equals the corresponding slice of the global mask
    sub = R.dropped(99, 0.25, 2, 4, qp[128:256], kp[64:192])
    assert torch.equal(sub, d1[:, :, 128:256, 64:192])


def test_cache_idx_decode_positions():
    """q replicated at cache_idx, KV cache sharded: equals dense attention over the cache prefix."""
    B, H, D, S, world = 1, 2, 16, 128, 4
    g = torch.Generator().manual_seed(5)
    k, v = [torch.randn(B, S, H, D, generator=g, dtype=torch.float64) for _ in range(2)]
    q = torch.randn(B, 8, H, D, generator=g, dtype=torch.float64)
    cache_idx = 77
    kw = dict(causal_block_size=1, query_chunk_size=8, key_chunk_size=16)

    def body(comm):
        sl = slice(comm.rank * 32, (comm.rank + 1) * 32)
        return R.ring_attention_ref(q, k[:, sl], v[:, sl], None, None, cache_idx, comm, True, kw)

    outs = run_fake_ring(world, body)
    ref = R.dense_attention(q, k, v, torch.arange(cache_idx, cache_idx + 8), torch.arange(S),
                            causal_block_size=1)
    for o in outs:
        assert torch.allclose(o, ref, atol=1e-10)


def test_inference_op_matches_masked_dense():
    B, H, D, S, world = 2, 2, 16, 96, 3
    g = torch.Generator().manual_seed(6)
    k, v = [torch.randn(B, S, H, D, generator=g, dtype=torch.float64) for _ in range(2)]
    q = torch.randn(B, 1, H, D, generator=g, dtype=torch.float64, requires_grad=True)
    mask = torch.zeros(B, 1, 1, S, dtype=torch.bool)
    mask[0, ..., :50] = True
    mask[1, ..., :91] = True

    def body(comm):
        sl = slice(comm.rank * 32, (comm.rank + 1) * 32)
        return R.RingAttentionInferenceRef.apply(q, k[:, sl], v[:, sl], mask, comm, True)

    outs = run_fake_ring(world, body)
    ref = R.dense_attention(q, k, v, extra_masked=~mask)
    for o in outs:
        assert torch.allclose(o, ref, atol=1e-10)


def test_merge_partials_equals_joint_softmax():
    q, k, v = _rand(1, 16, 2, 8, seed=7)
    oa, la = R.dense_attention(q, k[:, :6], v[:, :6], return_lse=True)
    ob, lb = R.dense_attention(q, k[:, 6:], v[:, 6:], return_lse=True)
    o, lse = R.merge_partials(oa, la, ob, lb)
    ref, ref_lse = R.dense_attention(q, k, v, return_lse=True)
    assert torch.allclose(o, ref, atol=1e-10) and torch.allclose(lse, ref_lse, atol=1e-10)


def test_fully_masked_rows_are_zero():
    q, k, v = _rand(1, 8, 1, 4, seed=8)
    out, lse = R.dense_attention(q, k, v, torch.arange(8), torch.arange(100, 108), causal_block_size=1,
                                 return_lse=True)
    assert torch.equal(out, torch.zeros_like(out)) and torch.isinf(lse).all()


def test_layout_roundtrip():
    x = torch.arange(2 * 64 * 3).view(2, 64, 3)
    for world in (1, 2, 4, 8):
        y = R.to_layout(x, world, "zigzag")
        assert torch.equal(R.from_layout(y, world, "zigzag"), x)
        if world > 1:
            pos = torch.cat([R.shard_positions(r, world, 64 // world, "zigzag") for r in range(world)])
            assert sorted(pos.tolist()) == list(range(64))


def test_explicit_pair_layout_on_the_ring():
    """Any pairing of the half-chunks is a valid layout: the ring against dense attention with a pairing that is
    neither contiguous nor zig-zag, causal and with segment ids."""
    _ring_case(4, "pairs:0-5,1-2,3-6,4-7", 1, seg=True, S=512, H=2, D=16, qc=64, dtype=torch.float64)
    with pytest.raises(ValueError):
        R.layout_pairs("pairs:0-1,1-2", 2)          # not a perfect matching
    with pytest.raises(ValueError):
        R.layout_pairs("pairs:0-1", 2)              # wrong number of pairs


def test_balanced_pairs_for_packed_documents():
    """Without document boundaries the balancing pairing is the zig-zag; with packed documents it lowers the
    largest per-rank work below the zig-zag's."""
    world, S = 4, 4096
    ids = torch.zeros(2, S, dtype=torch.int32)
    assert R.layout_pairs(R.balanced_pairs(ids, world), world) == R.layout_pairs("zigzag", world)

    def rank_work(seg, layout):
        pos = torch.arange(S).expand_as(seg)
        start_flag = torch.ones_like(seg, dtype=torch.bool)
        start_flag[:, 1:] = seg[:, 1:] != seg[:, :-1]
        start = torch.cummax(torch.where(start_flag, pos, torch.zeros_like(pos)), 1).values
        w = (pos - start + 1).double()
        return [float(w.index_select(1, R.shard_positions(r, world, S // world, layout)).sum()) for r in range(world)]

    g = torch.Generator().manual_seed(3)
    worse = 0
    for trial in range(8):
        seg = torch.cumsum((torch.rand(1, S, generator=g) < 1 / 300.0).int(), 1).int()
        lay = R.balanced_pairs(seg, world)
        wb, wz = rank_work(seg, lay), rank_work(seg, "zigzag")
        assert abs(sum(wb) - sum(wz)) < 1e-6 * sum(wz)      # the same total work, distributed differently
        assert max(wb) <= max(wz) + 1e-9
        worse += max(wb) < 0.97 * max(wz)
    assert worse >= 4                                         # and usually clearly better
