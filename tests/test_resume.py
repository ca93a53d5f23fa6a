"""What the reference host's --load relies on (trainer.cpp:64-80, checkpoint.cpp:506-552): weights,
momentum, variance and the step read from one engine and written into a fresh one — in the order
tg_set_weights, tg_set_onecycle, tg_set_optimizer_state, tg_set_data — continue the run bit for bit
as if it had never stopped, with and without a OneCycle schedule, for both architectures, also
across the CUDA-graph replay of the step."""
import numpy as np
import pytest

from oracle.model import Arch, Model
from turbogpt_b200 import Config, ConfigEx, Native, bridge

pytestmark = pytest.mark.gpu


def _engine(kind, flags=0):
    if kind == "reference":
        return Native(Config(depth=4, context=8, batch=16)), Model(Arch.reference(4), scale=.05).flat()
    base = Config(depth=2, context=128, batch=4, learning_rate=1e-3, clip=1.0)
    ex = ConfigEx.gpt(base, 128, 2, flags=flags)
    return Native(ex), bridge.initialize_weights(ex)


@pytest.mark.parametrize("kind", ["reference", "gpt"])
@pytest.mark.parametrize("scheduled", [False, True])
def test_resumed_run_equals_uninterrupted_run(kind, scheduled):
    data = np.random.default_rng(21).integers(0, 64, 1 << 14, dtype=np.uint8)
    total, first = 8, 4

    def start(weights):
        engine, initial = _engine(kind)
        engine.set_weights(initial if weights is None else weights)
        if scheduled:
            engine.set_onecycle(total)
        return engine

    whole = start(None)
    whole.set_data(data)
    whole.train(total)
    whole_losses = whole.training_losses(total)
    expected = whole.weights(), *whole.optimizer_state()
    whole.close()

    head = start(None)
    head.set_data(data)
    head.train(first)
    head_losses = head.training_losses(first)
    weights, (momentum, variance, step) = head.weights(), head.optimizer_state()
    head.close()
    assert step == first

    tail = start(weights)
    tail.set_optimizer_state(momentum, variance, step)
    tail.set_data(data)
    tail.train(total - first)
    tail_losses = tail.training_losses(total - first)
    actual = tail.weights(), *tail.optimizer_state()
    if scheduled:  # the schedule ends where the uninterrupted run's did
        assert tail.lib.tg_train(tail.handle, 1) < 0 and b"OneCycle" in tail.lib.tg_error()
    tail.close()

    np.testing.assert_array_equal(np.concatenate([head_losses, tail_losses]), whole_losses)
    np.testing.assert_array_equal(actual[0], expected[0])
    np.testing.assert_array_equal(actual[1], expected[1])
    np.testing.assert_array_equal(actual[2], expected[2])
    assert actual[3] == expected[3] == total
