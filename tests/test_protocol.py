"""Model-checks the symmetric-memory schedules (KV slots, slabs, dK/dV accumulators, decode inbox)
over every interleaving the barriers allow, and checks that the checker notices broken variants."""
import pytest

from ringattention_b200.parallel import protocol as P


@pytest.mark.parametrize("n", [2, 3])
def test_forward_schedule_is_race_free(n):
    progs = [P.ring_forward_program(r, n, calls=3) for r in range(n)]
    assert P.check_schedule(progs) is None


def test_forward_without_double_buffering_races():
    progs = [P.ring_forward_program(r, 2, calls=2, double_buffer=False) for r in range(2)]
    assert "stage" in (P.check_schedule(progs) or "")


def test_forward_without_barrier_races():
    progs = [P.ring_forward_program(r, 2, calls=1, barrier=False) for r in range(2)]
    assert P.check_schedule(progs) is not None


@pytest.mark.parametrize("n", [2, 3])
def test_backward_schedule_is_race_free(n):
    progs = [P.ring_backward_program(r, n, calls=2) for r in range(n)]
    assert P.check_schedule(progs) is None


def test_backward_needs_its_second_barrier():
    progs = [P.ring_backward_program(r, 2, calls=1, second_barrier=False) for r in range(2)]
    assert "cast" in (P.check_schedule(progs) or "") or "acc" in (P.check_schedule(progs) or "")


@pytest.mark.parametrize("n", [2, 3])
def test_decode_inbox_is_race_free(n):
    progs = [P.decode_program(r, n, calls=3) for r in range(n)]
    assert P.check_schedule(progs) is None


def test_decode_single_buffer_races():
    progs = [P.decode_program(r, 2, calls=2, double_buffer=False) for r in range(2)]
    assert P.check_schedule(progs) is not None
