"""The training-state file for any architecture (tg_ex_save_checkpoint / tg_ex_load_checkpoint):
round trip, torch.load, refusal of a file written for other dimensions, and — where the reference's
own reader was built (oracle/_ref/ckpt_probe, `make -C oracle ref`) — that a file of the reference
architecture loads in the reference's checkpoint.cpp and that a file the reference wrote loads here."""
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from turbogpt_b200 import Config, ConfigEx, bridge

PROBE = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "ckpt_probe"


def _state(config, seed=0):
    rng = np.random.default_rng(seed)
    count = bridge.load_library().tg_ex_parameter_count(config)
    schedule = bridge.OneCycle(40)
    return dict(weights=rng.standard_normal(count).astype(np.float32),
                momentum=rng.standard_normal(count).astype(np.float32),
                variance=rng.random(count).astype(np.float32), step=17, schedule=schedule, train_seconds=12.5,
                final_loss_sums=rng.random(config.base.context), final_loss_batches=0)


def _same(loaded, state):
    for key in ("weights", "momentum", "variance", "final_loss_sums"):
        np.testing.assert_array_equal(loaded[key], state[key])
    assert loaded["step"] == state["step"] and loaded["final_loss_batches"] == state["final_loss_batches"]
    assert loaded["train_seconds"] == state["train_seconds"]
    assert loaded["schedule"].total_steps == state["schedule"].total_steps
    assert loaded["schedule"].warmup_fraction == state["schedule"].warmup_fraction


def test_round_trip_and_torch_load(tmp_path):
    config = ConfigEx.gpt(Config(depth=2, context=64, batch=4), 128, 2, 384)
    state = _state(config)
    path = tmp_path / "model.pt"
    bridge.save_checkpoint(path, config, **state)
    _same(bridge.load_checkpoint(path, config), state)
    loaded = torch.load(path, map_location="cpu", weights_only=True)
    assert set(loaded) == {"model", "opt", "lr_scheduler", "trainer"}
    np.testing.assert_array_equal(loaded["model"]["weights"].numpy(), state["weights"])
    np.testing.assert_array_equal(loaded["opt"]["momentum"].numpy(), state["momentum"])
    np.testing.assert_array_equal(loaded["opt"]["variance"].numpy(), state["variance"])
    assert int(loaded["model"]["depth"]) == 2 and int(loaded["model"]["context"]) == 64
    assert loaded["model"]["architecture"].tolist() == [128, 2, 384, 1, 1, 1, 1, 0, 1]
    assert int(loaded["opt"]["step"]) == 17 and int(loaded["lr_scheduler"]["total_steps"]) == 40
    assert float(loaded["trainer"]["train_seconds"]) == 12.5
    np.testing.assert_array_equal(loaded["trainer"]["final_loss_sums"].numpy(), state["final_loss_sums"])


def test_other_dimensions_are_refused(tmp_path):
    config = ConfigEx.gpt(Config(depth=2, context=64, batch=4), 128, 2, 384)
    path = tmp_path / "model.pt"
    bridge.save_checkpoint(path, config, **_state(config))
    for other in (ConfigEx.gpt(Config(depth=2, context=64, batch=4), 128, 4, 384),     # heads
                  ConfigEx.gpt(Config(depth=3, context=64, batch=4), 128, 2, 384),     # depth
                  ConfigEx.gpt(Config(depth=2, context=32, batch=4), 128, 2, 384),     # context
                  ConfigEx.reference(Config(depth=2, context=64, batch=4))):           # architecture
        with pytest.raises(RuntimeError, match="mismatch|bytes"):
            bridge.load_checkpoint(path, other)
    damaged = bytearray(path.read_bytes())
    damaged[len(damaged) // 2] ^= 0x40
    (tmp_path / "damaged.pt").write_bytes(damaged)
    with pytest.raises(RuntimeError, match="checksum"):
        bridge.load_checkpoint(tmp_path / "damaged.pt", config)


@pytest.mark.skipif(not PROBE.exists(), reason="the reference's reader was not built (make -C oracle ref)")
def test_reference_reader_and_writer_interoperate(tmp_path):
    """ckpt_probe links the reference's unmodified checkpoint.cpp: `load` prints what its
    load_training_state read from a file, `save` writes a file with its save_training_state."""
    config = ConfigEx.reference(Config(depth=4, context=8, batch=16))
    state = _state(config)
    ours = tmp_path / "ours.pt"
    bridge.save_checkpoint(ours, config, **state)
    printed = subprocess.check_output([str(PROBE), "load", str(ours), "4", "8"], text=True).split()
    assert int(printed[0]) == state["step"] and int(printed[1]) == 40
    assert float(printed[2]) == pytest.approx(float(state["weights"].astype(np.float64).sum()), rel=1e-12)
    assert float(printed[3]) == pytest.approx(float(state["momentum"].astype(np.float64).sum()), rel=1e-12)
    theirs = tmp_path / "theirs.pt"
    subprocess.check_call([str(PROBE), "save", str(theirs), "4", "8", "11"])
    loaded = bridge.load_checkpoint(theirs, config)   # no architecture record: the reference architecture
    assert loaded["step"] == 11 and loaded["schedule"].total_steps == 40
    np.testing.assert_array_equal(loaded["weights"], np.arange(len(loaded["weights"]), dtype=np.float32) * .001)
    with pytest.raises(RuntimeError, match="mismatch|bytes"):
        bridge.load_checkpoint(theirs, ConfigEx.gpt(Config(depth=4, context=8, batch=16), 16, 4, 48))
