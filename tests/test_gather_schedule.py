"""Host-side schedule of the FSDP weight gather: residency, prefetch prediction and its safety
rules, checked on the call sequence of a training step (no GPU involved)."""
from ringattention_b200.models.params import GatherSchedule

KINDS = ("wqkv", "wo", "wgu", "wd", "lm_head")


def _step_sequence(layers, chunks=4):
    seq = []
    for l in range(layers):
        seq += [f"l{l}.wqkv", f"l{l}.wo"] + [f"l{l}.wgu", f"l{l}.wd"] * chunks
    seq += ["lm_head", "lm_head"] * chunks
    for l in reversed(range(layers)):
        seq += [f"l{l}.wqkv", f"l{l}.wo"] + [f"l{l}.wgu", f"l{l}.wd", f"l{l}.wgu"] * chunks
        seq += [f"l{l}.wo", f"l{l}.wqkv"]
    return seq


def _run_step(s, seq):
    """Replays one step and checks the invariants of every call."""
    for name in seq:
        plan = s.plan(name)
        regs = s.regions[s.kind(name)]
        assert regs[plan["region"]][0] == name
        assert regs[plan["region"]][1] == plan["target"] <= s.flag_base
        if plan["prefetch"] is not None:
            nm2, r2, t2 = plan["prefetch"]
            assert plan["copy_ctas"] == s.gather_ctas and t2 == s.flag_base
            # the copy never lands in the region this very call reads
            assert not (s.kind(nm2) == s.kind(name) and r2 == plan["region"])
            assert s.regions[s.kind(nm2)][r2][0] == nm2
    s.invalidate()


def test_first_step_gathers_later_steps_prefetch():
    s = GatherSchedule(KINDS, gather_ctas=16)
    seq = _step_sequence(layers=4)
    _run_step(s, seq)
    first = dict(s.stats)
    assert first["prefetches"] == 0 and first["gathers"] + first["resident_calls"] == len(seq)
    _run_step(s, seq)
    second = {k: s.stats[k] - first[k] for k in first}
    # only the cold start of the step (nothing resident to ride on) still gathers inside a waiting call
    assert second["gathers"] <= 4 and second["prefetches"] >= first["gathers"] - 4 - 1
    assert second["gathers"] + second["resident_calls"] == len(seq)


def test_a_diverging_step_stops_predicting_but_stays_consistent():
    s = GatherSchedule(KINDS, gather_ctas=8)
    _run_step(s, _step_sequence(layers=3))
    before = dict(s.stats)
    other = ["l0.wqkv", "l2.wd", "l1.wo", "l2.wd", "lm_head", "l0.wqkv"]
    _run_step(s, other)
    assert s.stats["prefetches"] - before["prefetches"] <= 1  # at most the one issued before the divergence
    assert s.trace_prev == other


def test_prefetch_can_be_switched_off():
    s = GatherSchedule(KINDS, gather_ctas=8, prefetch=False)
    seq = _step_sequence(layers=2)
    _run_step(s, seq)
    _run_step(s, seq)
    assert s.stats["prefetches"] == 0
