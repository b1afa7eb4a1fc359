"""sm_100a attention kernels (one ring step) against the fp32 dense oracle, plus the public op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, Sq, Sk, H, D, cbs=0, q_off=0, k_off=0, seg=False, bias=False, pdrop=0.0, prev=False, seg_p=0.01):
    from ringattention_b200.ops import _lib, flash, reference as R

    torch.manual_seed(0)
    dev = "cuda"
    q = torch.randn(B, Sq, H, D, device=dev).bfloat16()
    k = torch.randn(B, Sk, H, D, device=dev).bfloat16()
    v = torch.randn(B, Sk, H, D, device=dev).bfloat16()
    do = torch.randn(B, Sq, H, D, device=dev).bfloat16()
    qp, kp = flash.Positions(q_off), flash.Positions(k_off)
    q_pos, k_pos = qp.tensor(Sq, dev), kp.tensor(Sk, dev)
    ms = flash.MaskSpec(causal_block_size=cbs, q_pos=qp, k_pos=kp)
    seg_q = seg_k = bs = None
    if seg:
        tot = max(q_off + Sq, k_off + Sk)
        ids = torch.cumsum((torch.rand(B, tot, device=dev) < seg_p).int(), dim=1).int()
        seg_q, seg_k = ids[:, q_pos].contiguous(), ids[:, k_pos].contiguous()
        ms.seg_q, ms.seg_k = seg_q, seg_k
        ms.seg_q_mm, ms.seg_k_mm = flash.seg_tile_minmax(seg_q), flash.seg_tile_minmax(seg_k)
    if bias:
        bs = torch.randn(B, 1, Sk, device=dev)
        ms.bias = bs
    if pdrop > 0:
        ms.seed, ms.pdrop = 1234567891234, pdrop
    o_prev = lse_prev = None
    if prev:
        o_prev = torch.randn(B, Sq, H, D, device=dev)
        lse_prev = torch.randn(B, H, Sq, device=dev)
    out, lse = flash.flash_fwd(q, k, v, ms, o_prev=o_prev, lse_prev=lse_prev, out_fp32=prev)
    qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref, ref_lse = R.dense_attention(qf, kf, vf, q_pos, k_pos, causal_block_size=cbs or None,
                                     bias=None if bs is None else bs[:, :, None, :], seg_q=seg_q,
                                     seg_k=seg_k, seed=ms.seed, pdrop=pdrop, dtype=torch.float32,
                                     return_lse=True)
    if prev:
        mref, mlse = R.merge_partials(o_prev, lse_prev, ref.detach(), ref_lse.detach())
        assert (out.float() - mref).abs().max() < 0.02
        return
    assert (out.float() - ref.detach()).abs().max() < 0.02
    fin = torch.isfinite(ref_lse)
    if fin.any():
        assert (lse[fin] - ref_lse.detach()[fin]).abs().max() < 1e-2
    assert bool((lse[~fin] == float("-inf")).all())
    # backward
    lse2, delta = flash.flash_bwd_prep(out, do, lse)
    dq_acc = torch.zeros(B, Sq, H, D, device=dev)
    dk, dv = torch.zeros_like(k), torch.zeros_like(k)
    flash.flash_bwd(q, k, v, do, lse2, delta, ms, dq_acc, dk, dv)
    torch.cuda.synchronize()
    _lib.check_status()
    ref.backward(do.float())
    for got, want in ((dq_acc, qf.grad), (dk, kf.grad), (dv, vf.grad)):
        assert (got.float() - want).abs().max() <= 0.02 * want.abs().max() + 1e-3


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("cbs", [0, 1, 64])
def test_attention_causal_variants(D, cbs):
    _case(2, 512, 512, 2, D, cbs=cbs)


def test_attention_ragged_and_offsets():
    _case(1, 200, 333, 2, 128)
    _case(1, 200, 333, 2, 128, cbs=1, q_off=133)
    _case(1, 384, 640, 2, 128, cbs=1, q_off=256)
    _case(1, 300, 700, 3, 64, cbs=1, q_off=400, seg=True)


def test_attention_segments_bias_dropout():
    _case(1, 512, 512, 2, 128, cbs=1, seg=True)
    _case(1, 512, 512, 2, 128, bias=True)
    _case(1, 512, 512, 2, 128, cbs=1, pdrop=0.2)


def test_attention_long_documents_take_the_plain_path_inside_a_segment():
    """Documents several tiles long: tile pairs inside one segment skip the per-column masking, pairs of
    different segments are skipped through the visibility bitmask, boundary tiles take the masked path."""
    _case(2, 2048, 2048, 2, 128, cbs=1, seg=True, seg_p=0.002)
    _case(1, 1536, 2048, 2, 128, cbs=0, seg=True, seg_p=0.003)
    _case(1, 1024, 1024, 2, 64, cbs=1, seg=True, seg_p=0.004, pdrop=0.1)


def test_attention_fully_masked_block_and_carry():
    _case(1, 512, 512, 2, 128, cbs=1, k_off=512)           # block entirely in the causal future
    _case(1, 512, 512, 2, 128, cbs=1, q_off=512, prev=True)  # merge with an earlier ring step


def test_public_op_autograd_matches_reference():
    import ringattention_b200 as rab

    torch.manual_seed(3)
    q, k, v = [torch.randn(2, 384, 4, 128, device="cuda").bfloat16().requires_grad_(True) for _ in range(3)]
    ids = torch.cumsum((torch.rand(2, 384, device="cuda") < 0.02).int(), 1).int()
    kw = dict(causal_block_size=1, query_chunk_size=128, key_chunk_size=128)
    out = rab.ringattention(q, k, v, None, ids, None, None, True, kw)
    g = torch.randn_like(out)
    out.backward(g)
    q2, k2, v2 = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = rab.ringattention_ref(q2, k2, v2, None, ids, None, None, True, kw)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 0.02
    for a, b in ((q.grad, q2.grad), (k.grad, k2.grad), (v.grad, v2.grad)):
        assert (a.float() - b).abs().max() <= 0.02 * b.abs().max() + 1e-3


def test_full_bias_is_served_by_the_torch_path():
    import ringattention_b200 as rab

    q, k, v = [torch.randn(1, 64, 2, 64, device="cuda").bfloat16() for _ in range(3)]
    bias = torch.randn(1, 1, 64, 64, device="cuda")
    out = rab.ringattention(q, k, v, bias, None, None, None, True, dict(query_chunk_size=32, key_chunk_size=32))
    assert out.shape == q.shape and out.dtype == v.dtype
