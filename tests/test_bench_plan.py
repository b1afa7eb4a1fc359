"""Step counts that bench.py fits into its wall-clock budget."""
import importlib.util
import os

import pytest

_spec = importlib.util.spec_from_file_location(
    "bench_module", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
bench = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bench)


def test_everything_fits():
    assert bench.plan_counts(5, 20, 1, 1.0, 1000.0) == (4, 20, 20)
    assert bench.plan_counts(5, 20, 1, 1.0, float("inf")) == (4, 20, 20)


def test_long_steps_keep_floors():
    # 60 s steps, 430 s left after the first warm-up step: 2 more warm-up, 3 timed, 2 end to end
    assert bench.plan_counts(5, 20, 1, 60.0, 430.0) == (2, 3, 2)
    # after three warm-up steps, 48 s steps, 334 s left: the spare step goes to the timed region
    assert bench.plan_counts(3, 20, 3, 48.0, 334.0) == (0, 4, 2)


def test_warmup_gives_way_last():
    # only 5 steps fit: the timed and end-to-end floors stay, warm-up stops at the one step already run
    assert bench.plan_counts(5, 20, 1, 60.0, 300.0) == (0, 3, 2)
    # nothing fits: the floors are run all the same
    assert bench.plan_counts(5, 20, 1, 600.0, 10.0) == (0, 3, 2)


@pytest.mark.parametrize("steps", [1, 2])
def test_small_requests_are_not_raised(steps):
    w, k, e = bench.plan_counts(0, steps, 0, 1.0, 1000.0)
    assert (w, k, e) == (0, steps, steps)


def test_tp_mesh_is_refused():
    from ringattention_b200.config import LlamaConfig, MeshConfig, TrainConfig
    from ringattention_b200.trainer import Trainer

    assert MeshConfig.parse("1,1,2,1").tp == 2  # expressible ...
    with pytest.raises(ValueError, match="tensor parallelism"):  # ... but not trainable
        Trainer(LlamaConfig.named("llama-tiny"), TrainConfig(model="llama-tiny", mesh="1,1,2,1"))
