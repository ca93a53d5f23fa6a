"""The new engine beside the reference's own CUDA engine on the same GPU, same weights, same bytes.
The reference engine is the reference's cuda/runtime.cu + cuda/engine_state.cu compiled unmodified for
sm_100 by `make -C oracle ref` into oracle/_ref/ (test infrastructure, not shipped); both libraries are
driven through the same ctypes signatures.  Skipped where that build is absent."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from oracle.model import Arch, Model
from turbogpt_b200 import Config, Native, bridge
from helpers import relative

pytestmark = pytest.mark.gpu
REFERENCE = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libturbogpt_ref.so"


@pytest.fixture(scope="module")
def reference_library():
    if not REFERENCE.exists():
        pytest.skip("reference engine not built (make -C oracle ref)")
    return bridge.declare_reference_interface(C.CDLL(str(REFERENCE)))


# batch * context / 32 tiles must fill the reference's resident blocks evenly (cuda/runtime.cu:17-29)
@pytest.mark.parametrize("depth,context,batch", [(4, 4, 16), (8, 8, 16), (4, 8, 32)])
def test_forward_and_gradients_match_the_reference_engine(reference_library, depth, context, batch):
    cfg = Config(depth=depth, context=context, batch=batch)
    weights = Model(Arch.reference(depth), scale=.08).flat()
    rng = np.random.default_rng(71)
    x = rng.integers(0, 256, (batch, context), dtype=np.uint8)
    y = rng.integers(0, 256, x.shape, dtype=np.uint8)
    results = []
    for library in (reference_library, None):
        with Native(cfg, library=library) as engine:
            engine.set_weights(weights)
            results.append(engine.batch(x, y))
    (ref_logits, ref_grad, ref_losses), (logits, grad, losses) = results
    # Same rounding points; only accumulation order and fast-math differ (verify.py's own bounds).
    assert relative(logits, ref_logits) < .005
    assert relative(grad, ref_grad) < .01
    np.testing.assert_allclose(losses, ref_losses, atol=.003, rtol=.001)
    assert np.mean(logits == ref_logits) > .9  # BF16 logits are bit-identical almost everywhere


def test_training_steps_match_the_reference_engine(reference_library):
    """Eight full steps (device sampling, Muon + AdamW, OneCycle) from the same state."""
    cfg = Config(depth=4, context=4, batch=32)
    weights = Model(Arch.reference(4), scale=.05).flat()
    data = np.random.default_rng(4).integers(0, 256, 4096, dtype=np.uint8)
    out = []
    for library in (reference_library, None):
        with Native(cfg, library=library) as engine:
            engine.set_weights(weights)
            engine.check(engine.lib.tg_set_data(engine.handle, data.ctypes.data, len(data)))
            engine.check(engine.lib.tg_set_onecycle(engine.handle, C.byref(bridge.OneCycle(8))))
            engine.check(engine.lib.tg_train(engine.handle, 8))
            losses = np.empty((8, cfg.context), np.float32)
            engine.check(engine.lib.tg_get_training_losses(engine.handle, losses.ctypes.data, 8))
            out.append((losses, engine.weights()))
    (ref_losses, ref_weights), (losses, new_weights) = out
    np.testing.assert_allclose(losses[0], ref_losses[0], atol=1e-4)  # same bytes sampled, same model
    np.testing.assert_allclose(losses, ref_losses, atol=.01, rtol=.002)
    assert relative(new_weights - weights, ref_weights - weights) < .1  # BF16 Newton-Schulz noise
    mask = np.load(Path(__file__).parent / "golden" / "optimizer.npz")["adam_mask"]
    # eight steps compound the last-bit differences of the BF16 gradients (Muon feeds them back)
    assert relative(new_weights[mask] - weights[mask], ref_weights[mask] - weights[mask]) < .05
