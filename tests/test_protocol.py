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


@pytest.mark.parametrize("n", [2, 3])
def test_fsdp_weight_gather_is_race_free(n):
    from ringattention_b200.parallel.protocol import check_schedule, fsdp_program

    assert check_schedule([fsdp_program(r, n, steps=2) for r in range(n)]) is None


def test_fsdp_needs_the_collectives_around_the_update():
    from ringattention_b200.parallel.protocol import check_schedule, fsdp_program

    # without the sync after the optimizer a peer's next step may read a shard that is being rewritten
    assert check_schedule([fsdp_program(r, 2, steps=2, sync_after_update=False) for r in range(2)]) is not None
    # without the gradient collective a rank may rewrite its shard while a slower peer still reads it
    assert check_schedule([fsdp_program(r, 2, steps=1, reduce_before_update=False) for r in range(2)]) is not None


@pytest.mark.parametrize("n,rows", [(2, 2), (3, 2), (2, 3)])
def test_row_exchange_with_two_slots_is_race_free(n, rows):
    assert P.check_row_exchange(n, rows, launches=4) is None


def test_row_exchange_with_one_slot_overwrites_unmerged_rows():
    assert "overwrites" in (P.check_row_exchange(2, 2, launches=2, slots=1) or "")
