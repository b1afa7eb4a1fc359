"""Decode path: split-KV kernel + merge against the dense oracle, small-M linear, and the
inference engine (chunked prefill + greedy decode) against a full PyTorch forward."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 1, 4, 128, 3000), (2, 4, 3, 64, 1111), (1, 8, 2, 128, 700), (1, 3, 2, 128, 500)])
def test_decode_attention_matches_dense(shape):
    import ringattention_b200 as rab
    from ringattention_b200.ops import _lib, decode as Dk, reference as R
    from ringattention_b200.parallel.mesh import resolve_axis

    B, QL, H, D, S = shape
    torch.manual_seed(0)
    q = torch.randn(B, QL, H, D, device="cuda").bfloat16()
    k = torch.randn(B, S, H, D, device="cuda").bfloat16()
    v = torch.randn_like(k)
    mask = torch.rand(B, 1, QL, S, device="cuda") < 0.7
    out = rab.ringattention_inference(q, k, v, mask, None)
    ref = R.dense_attention(q, k, v, extra_masked=~mask, dtype=torch.float32)
    assert (out.float() - ref).abs().max() < 0.02
    # position-driven variant used by the decoding loop: causal rule + partially filled cache
    out2 = Dk.ring_decode_attention(q, k, v, None, resolve_axis(None), n_valid=S - 100, q_pos0=S - 200, k_pos0=0)
    ref2 = R.dense_attention(q, k[:, :S - 100], v[:, :S - 100], torch.arange(S - 200, S - 200 + QL, device="cuda"),
                             torch.arange(S - 100, device="cuda"), causal_block_size=1, dtype=torch.float32)
    assert (out2.float() - ref2).abs().max() < 0.02
    torch.cuda.synchronize()
    _lib.check_status()


def test_decode_fully_masked_rows_are_zero():
    import ringattention_b200 as rab

    q = torch.randn(1, 2, 2, 128, device="cuda").bfloat16()
    k = torch.randn(1, 300, 2, 128, device="cuda").bfloat16()
    mask = torch.zeros(1, 1, 2, 300, dtype=torch.bool, device="cuda")
    mask[0, 0, 1, :17] = True
    out = rab.ringattention_inference(q, k, k, mask, None)
    assert bool((out[:, 0] == 0).all()) and bool(torch.isfinite(out.float()).all())


def test_small_m_linear():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(1)
    for M in (1, 3, 8):
        x = torch.randn(M, 512, device="cuda").bfloat16()
        w = torch.randn(1000, 512, device="cuda").bfloat16()
        r = torch.randn(M, 1000, device="cuda").bfloat16()
        y = K.small_m_linear(x, w, residual=r)
        ref = x.float() @ w.float().t() + r.float()
        assert (y.float() - ref).abs().max() <= 0.01 * ref.abs().max() + 0.05


def test_small_m_linear_prologues():
    """RMSNorm and SwiGLU applied while the kernel reads x, against plain fp32 PyTorch."""
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(2)
    for M in (1, 4, 8):
        x = torch.randn(M, 1024, device="cuda").bfloat16()
        g = (1 + 0.1 * torch.randn(1024, device="cuda")).bfloat16()
        w = (torch.randn(776, 1024, device="cuda") / 32).bfloat16()
        y = K.norm_linear(x, g, 1e-5, w)
        xf = x.float()
        ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()) @ w.float().t()
        assert (y.float() - ref).abs().max() <= 0.01 * ref.abs().max() + 0.02

        gu = torch.randn(M, 2 * 1024, device="cuda").bfloat16()
        r = torch.randn(M, 776, device="cuda").bfloat16()
        y = K.swiglu_linear(gu, w, residual=r)
        h = (torch.nn.functional.silu(gu[:, :1024].float()) * gu[:, 1024:].float()).bfloat16().float()
        ref = h @ w.float().t() + r.float()
        assert (y.float() - ref).abs().max() <= 0.01 * ref.abs().max() + 0.02
        # the same numbers as the two-launch path: the activation is rounded to bf16 in both
        two = K.small_m_linear(K.swiglu_fwd(gu), w, residual=r)
        assert torch.equal(y, two)


@pytest.mark.parametrize("D,striped", [(128, False), (64, True)])
def test_rope_append_equals_rope_then_append(D, striped):
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(3)
    B, H, S_max = 2, 8, 64
    qkv = torch.randn(B, 1, 3, H, D, device="cuda").bfloat16()
    state = torch.tensor([37, 0], device="cuda", dtype=torch.int64)
    stripe = (2, 1, 16, 32) if striped else None  # decoded token 5 -> rank 1, row 16 + 2
    caches = [torch.zeros(B, 2, H, S_max, D, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    views = [(c[:, 0].transpose(1, 2), c[:, 1].transpose(1, 2)) for c in caches]
    a = qkv.clone()
    K.rope_at_(a.view(B, 1, 3 * H, D)[:, :, :2 * H], state, 10000.0)
    K.kv_append(a, views[0][0], views[0][1], state, stripe=stripe)
    b = qkv.clone()
    K.rope_append(b, views[1][0], views[1][1], state, 10000.0, stripe=stripe)
    assert torch.equal(a, b) and torch.equal(caches[0], caches[1])
    row = 18 if striped else 37
    assert torch.equal(views[1][0][:, row], b[:, 0, 1]) and torch.equal(views[1][1][:, row], b[:, 0, 2])
    written = int(torch.count_nonzero(views[1][0][:, row])) + int(torch.count_nonzero(views[1][1][:, row]))
    assert int(torch.count_nonzero(caches[1])) == written  # no other cache row was touched


def test_merge_exchange_gives_up_on_a_silent_peer_and_still_merges_its_own_rows():
    """The one-launch cross-GPU merge with a second "rank" that never signals (its buffers are local and nobody
    writes them): every row's wait runs out, the status word gets the peer-timeout code, the kernel returns and
    the context keeps working. The silent rank's inbox slots hold lse = -inf, so the merged rows equal this
    rank's own."""
    import ctypes

    from ringattention_b200.ops import _lib
    from ringattention_b200.ops import decode as Dk

    torch.manual_seed(4)
    rows, parts, D, n = 16, 3, 128, 2
    o_part = torch.randn(rows, parts, D, device="cuda")
    lse_part = torch.randn(rows, parts, device="cuda")
    boxes_o = torch.zeros(n, 2, rows, n, D, device="cuda")
    boxes_l = torch.full((n, 2, rows, n), float("-inf"), device="cuda")
    flags = torch.zeros(n, rows, n, dtype=torch.int32, device="cuda")
    sync = torch.zeros(2, dtype=torch.int32, device="cuda")
    tab = lambda t: torch.tensor([t[i].data_ptr() for i in range(n)], dtype=torch.int64, device="cuda")
    to, tl, tf = tab(boxes_o), tab(boxes_l), tab(flags)
    out = torch.empty(rows, D, device="cuda")
    st = _lib.status_tensor()
    st.zero_()
    vp = ctypes.c_void_p
    _lib.call("ra_decode_merge_exchange", vp(o_part.data_ptr()), vp(lse_part.data_ptr()),
              ctypes.c_longlong(parts * D), ctypes.c_longlong(D), ctypes.c_longlong(parts), ctypes.c_longlong(1),
              rows, parts, D, 1, 0, vp(out.data_ptr()), 1, vp(to.data_ptr()), vp(tl.data_ptr()),
              vp(boxes_o[0].data_ptr()), vp(boxes_l[0].data_ptr()), rows, vp(tf.data_ptr()), vp(sync.data_ptr()), n, 0,
              ctypes.c_ulonglong(50_000_000), vp(st.data_ptr()), _lib.stream_ptr())
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelError, match="peer flag"):
        _lib.check_status()
    assert sync.tolist() == [1, 0]  # the launch counter advanced, the arrival counter is back at zero
    w = torch.softmax(lse_part, dim=1)
    ref = (w[:, :, None] * o_part).sum(1)
    assert (out - ref).abs().max() < 1e-4
    assert Dk.exchange_fits(rows) and not Dk.exchange_fits(10 ** 6)


def test_cuda_core_kernels_still_serve_several_rows(monkeypatch):
    """Calls with 2-8 rows go to the tensor-core kernels by default; with the thresholds raised the CUDA-core
    kernels (which serve one row by default) take them and give the same answers."""
    from ringattention_b200.ops import decode as Dk, kernels as K, reference as R
    from ringattention_b200.parallel.mesh import resolve_axis

    torch.manual_seed(5)
    B, QL, H, D, S = 1, 4, 2, 128, 900
    q = torch.randn(B, QL, H, D, device="cuda").bfloat16()
    k = torch.randn(B, S, H, D, device="cuda").bfloat16()
    v = torch.randn_like(k)
    x = torch.randn(4, 1024, device="cuda").bfloat16()
    g = (1 + 0.1 * torch.randn(1024, device="cuda")).bfloat16()
    w = (torch.randn(520, 1024, device="cuda") / 32).bfloat16()
    outs = []
    for rows in (2, 9):
        monkeypatch.setattr(Dk, "MMA_MIN_ROWS", rows)
        monkeypatch.setattr(K, "LINEAR_MMA_MIN_ROWS", rows)
        o = Dk.ring_decode_attention(q, k, v, None, resolve_axis(None), n_valid=S, q_pos0=S - QL, k_pos0=0)
        outs.append((o.float(), K.norm_linear(x, g, 1e-5, w).float(), K.small_m_linear(x, w).float()))
    ref = R.dense_attention(q, k, v, torch.arange(S - QL, S, device="cuda"), torch.arange(S, device="cuda"),
                            causal_block_size=1, dtype=torch.float32)
    for o, _, _ in outs:
        assert (o - ref).abs().max() < 0.02
    assert (outs[0][1] - outs[1][1]).abs().max() <= 0.02 * outs[1][1].abs().max() + 0.02
    assert (outs[0][2] - outs[1][2]).abs().max() <= 0.01 * outs[1][2].abs().max() + 0.02


def test_prefill_and_greedy_decode_match_full_forward():
    from ringattention_b200.config import LlamaConfig
    from ringattention_b200.models.llama_infer import LlamaInference
    from llama_torch import llama_forward_torch
    from ringattention_b200.ops import _lib

    cfg = LlamaConfig.named("llama-tiny")
    inf = LlamaInference(cfg, max_context=1024, batch=2, seed=5)
    T = 384
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (2, T), device="cuda")
    gen, timing = inf.generate(prompt, 8, chunk=128)
    _lib.check_status()
    W = {n: inf.params.w(n) for n in inf.params.index}
    logits = llama_forward_torch(cfg, W, torch.cat([prompt, gen], dim=1).int())
    ref_next = logits[:, T - 1:-1].argmax(-1)
    assert (ref_next == gen).float().mean() >= 0.9
    assert len(timing["decode_ms"]) == 8 and inf.length == T + 8


def test_graph_replayed_decode_equals_eager_decode():
    """The CUDA-graph decode path (device-side position/step) must emit the same tokens as the eager path."""
    from ringattention_b200.config import LlamaConfig
    from ringattention_b200.models.llama_infer import LlamaInference
    from ringattention_b200.ops import _lib

    cfg = LlamaConfig.named("llama-tiny")
    torch.manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda")
    a = LlamaInference(cfg, max_context=512, batch=2, seed=7)
    b = LlamaInference(cfg, max_context=512, batch=2, seed=7)
    ga, _ = a.generate(prompt, 12, chunk=128, use_graph=True)
    gb, _ = b.generate(prompt, 12, chunk=128, use_graph=False)
    _lib.check_status()
    assert a._graph is not None and b._graph is None
    assert torch.equal(ga, gb)
    assert int(a.state[0].item()) == a.length == 256 + 12


def test_engine_reuse_after_reset_matches_a_fresh_engine():
    from ringattention_b200.config import LlamaConfig
    from ringattention_b200.models.llama_infer import LlamaInference

    cfg = LlamaConfig.named("llama-tiny")
    torch.manual_seed(4)
    p1 = torch.randint(0, cfg.vocab_size, (1, 256), device="cuda")
    p2 = torch.randint(0, cfg.vocab_size, (1, 384), device="cuda")
    eng = LlamaInference(cfg, max_context=1024, batch=1, seed=9)
    eng.generate(p1, 6, chunk=128)
    g2, _ = eng.generate(p2, 6, chunk=128)          # resets, re-records the decode graph
    fresh, _ = LlamaInference(cfg, max_context=1024, batch=1, seed=9).generate(p2, 6, chunk=128)
    assert torch.equal(g2, fresh) and eng.length == 384 + 6


@pytest.mark.parametrize("ql,S,H,D", [(1, 700, 2, 128), (8, 1111, 3, 64), (100, 900, 2, 128), (2048, 1536, 2, 128)])
def test_inference_op_any_query_length_with_gradients(ql, S, H, D):
    """ringattention_inference with a random boolean mask (ringattention_inference.py:8-35) and its VJP (:38-64)
    against dense fp32 attention, for query lengths on both sides of the 8-row decode kernel."""
    import ringattention_b200 as rab
    from ringattention_b200.ops import _lib, reference as R

    B = 2
    torch.manual_seed(ql)
    q, k, v = [torch.randn(B, n, H, D, device="cuda").bfloat16().requires_grad_(True) for n in (ql, S, S)]
    do = torch.randn(B, ql, H, D, device="cuda").bfloat16()
    mask = torch.rand(B, 1, ql, S, device="cuda") < 0.6
    mask[..., 0] = True  # no fully masked row: the dense oracle would average over nothing
    out = rab.ringattention_inference(q, k, v, mask, None)
    out.backward(do)
    qf, kf, vf = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = R.dense_attention(qf, kf, vf, extra_masked=~mask, dtype=torch.float32)
    ref.backward(do.float())
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out.float() - ref).abs().max() < 0.02
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert (got.float() - want).abs().max() <= 0.02 * want.abs().max() + 1e-3
    # without gradients the short queries take the split-KV decode kernel: same numbers
    with torch.no_grad():
        out2 = rab.ringattention_inference(q, k, v, mask, None)
    assert (out2.float() - ref).abs().max() < 0.02


def test_mask_bitmaps_round_trip():
    from ringattention_b200.ops import flash

    torch.manual_seed(3)
    B, Hm, Sq, Sk = 2, 3, 77, 301
    m = torch.rand(B, Hm, Sq, Sk, device="cuda") < 0.5
    by_q, by_k = flash.pack_mask(m)
    bits = torch.arange(32, device="cuda")
    got_q = ((by_q.unsqueeze(-1) >> bits) & 1).bool().flatten(3)[..., :Sk]        # (B, Hm, Sq, Sk)
    got_k = ((by_k.unsqueeze(-1) >> bits) & 1).bool().flatten(3)[..., :Sq]        # (B, Hm, Sk, Sq)
    assert torch.equal(got_q, m)
    assert torch.equal(got_k, m.transpose(2, 3))
    # padding bits are zero
    assert int(((by_q.unsqueeze(-1) >> bits) & 1).flatten(3)[..., Sk:].sum()) == 0


@pytest.mark.parametrize("ql,cache_idx", [(128, 384), (100, 411), (1, 639)])
def test_cache_idx_on_the_fused_path(ql, cache_idx):
    """``cache_idx``: replicated queries that start at global position ``cache_idx`` against the cache
    (ringattention_jax.py:31-35), causal, on the fused kernels including gradients."""
    import ringattention_b200 as rab
    from ringattention_b200.ops import _lib, reference as R

    B, H, D, Sk = 2, 2, 128, 640
    torch.manual_seed(cache_idx)
    q = torch.randn(B, ql, H, D, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B, Sk, H, D, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B, Sk, H, D, device="cuda").bfloat16().requires_grad_(True)
    do = torch.randn(B, ql, H, D, device="cuda").bfloat16()
    kw = dict(causal_block_size=1, query_chunk_size=128, key_chunk_size=128)
    out = rab.ringattention(q, k, v, None, None, cache_idx, None, True, kw)
    out.backward(do)
    qf, kf, vf = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = R.dense_attention(qf, kf, vf, torch.arange(cache_idx, cache_idx + ql, device="cuda"),
                            torch.arange(Sk, device="cuda"), causal_block_size=1, dtype=torch.float32)
    ref.backward(do.float())
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out.float() - ref).abs().max() < 0.02
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert (got.float() - want).abs().max() <= 0.02 * want.abs().max() + 1e-3


def test_fallback_to_pytorch_path_warns_once():
    import warnings

    import ringattention_b200 as rab
    from ringattention_b200 import api

    api._WARNED.clear()
    q = torch.randn(1, 64, 2, 64, device="cuda")  # fp32: not served by the kernels
    kw = dict(causal_block_size=1, query_chunk_size=64, key_chunk_size=64)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        rab.ringattention(q, q, q, None, None, None, None, True, kw)
        rab.ringattention(q, q, q, None, None, None, None, True, kw)
    assert sum("PyTorch path" in str(x.message) for x in w) == 1


def test_streams_sharing_one_cached_context():
    """Three decode streams on one shared prefix (read once per step for all of them, private tails) against three
    single-stream engines that each cached the prefix themselves; teacher-forced, logits compared step by step."""
    from ringattention_b200.config import LlamaConfig
    from ringattention_b200.models.llama_infer import LlamaInference
    from ringattention_b200.ops import _lib

    cfg = LlamaConfig.named("llama-tiny")
    torch.manual_seed(4)
    prompt = torch.randint(0, cfg.vocab_size, (1, 384), device="cuda")
    shared = LlamaInference(cfg, max_context=1024, batch=1, seed=7, streams=3, max_new_tokens=16)
    logits = None
    for c0 in range(0, 384, 128):
        logits = shared.prefill_chunk(prompt[:, c0:c0 + 128])
    singles = []
    for _ in range(3):
        e = LlamaInference(cfg, max_context=1024, batch=1, seed=7)
        for c0 in range(0, 384, 128):
            e.prefill_chunk(prompt[:, c0:c0 + 128])
        singles.append(e)
    tok = logits[0].topk(3).indices                        # three different continuations
    worst = 0.0
    for _ in range(6):
        la = shared.decode_step(tok)                        # (3, vocab)
        lb = torch.cat([e.decode_step(tok[i:i + 1]) for i, e in enumerate(singles)], dim=0)
        worst = max(worst, ((la - lb).abs().max() / lb.abs().max()).item())
        tok = lb.argmax(dim=-1)
    torch.cuda.synchronize()
    _lib.check_status()
    assert worst < 0.03, worst
    # the graph-replayed path gives the same tokens as the eager one from here on
    shared._tok_buf.copy_(tok.to(torch.int32))
    eager = shared.decode_step(tok).argmax(dim=-1)
    assert eager.shape == (3,)
