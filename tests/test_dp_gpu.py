"""Data-parallel training on two GPUs through the C ABI (NCCL inside the engine): two ranks with
micro-batch B must follow one engine with batch 2B on the same corpus.  Skipped on one GPU."""
import ctypes as C
import numpy as np
import pytest
import torch

from turbogpt_b200 import Config, ConfigEx, Native, bridge
from helpers import relative

pytestmark = pytest.mark.gpu

SHAPE = dict(depth=2, width=128, heads=2, context=128)
BATCH, STEPS = 4, 4


def _fixture():
    base = Config(depth=SHAPE["depth"], context=SHAPE["context"], batch=BATCH, learning_rate=1e-3, clip=1.0)
    ex = ConfigEx.gpt(base, SHAPE["width"], SHAPE["heads"])
    weights = bridge.initialize_weights(ex)
    data = np.random.default_rng(2).integers(0, 32, 1 << 14, dtype=np.uint8)
    return weights, data


def _config(batch, device, flags, mode, **extra):
    base = Config(depth=SHAPE["depth"], context=SHAPE["context"], batch=batch, device=device, learning_rate=1e-3,
                  clip=1.0)
    return ConfigEx.gpt(base, SHAPE["width"], SHAPE["heads"], flags=flags,
                        precision=bridge.PRECISION_FP32 if mode == "fp32" else bridge.PRECISION_BF16,
                        hidden_optimizer=bridge.HIDDEN_MUON if mode == "muon" else bridge.HIDDEN_ADAMW, **extra)


def _rank(rank, world, ident, flags, mode, out):
    import os
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    weights, data = _fixture()
    ex = _config(BATCH, rank, flags, mode, world=world, rank=rank)
    C.memmove(ex.nccl_id, ident, 128)
    with Native(ex) as engine:
        engine.set_weights(weights)
        engine.set_data(data)
        engine.train(STEPS)
        losses = engine.training_losses(STEPS)
        out.put((rank, losses, engine.weights()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("flags,mode", [(0, "bf16"), (bridge.FLAG_BF16_GRADIENT_EXCHANGE, "bf16"), (0, "fp32"),
                                        (0, "muon")])
def test_two_ranks_follow_one_engine_with_the_global_batch(flags, mode):
    """FP32 gradient buckets (the default) and buckets cast to BF16 for the wire; the FP32 check mode,
    where every tensor must agree to FP32 summation order; Muon, whose Newton-Schulz iterations are
    sharded by layer over the ranks and all-gathered."""
    import torch.multiprocessing as mp
    lib = bridge.load_library()
    ident = (C.c_uint8 * 128)()
    assert lib.tg_ex_nccl_unique_id(ident) == 0, lib.tg_error()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, bytes(ident), flags, mode, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict()
    for _ in range(2):
        rank, losses, weights = out.get(timeout=300)
        results[rank] = (losses, weights)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    weights, data = _fixture()
    single = _config(2 * BATCH, 0, 0, mode)
    with Native(single) as engine:
        engine.set_weights(weights)
        engine.set_data(data)
        engine.train(STEPS)
        whole_losses, whole_weights = engine.training_losses(STEPS), engine.weights()
    np.testing.assert_array_equal(results[0][1], results[1][1])          # replicas stay identical
    np.testing.assert_allclose(results[0][0], results[1][0], rtol=1e-6)  # both report the global losses
    np.testing.assert_allclose(results[0][0], whole_losses, rtol=2e-3, atol=2e-3)
    # Newton-Schulz pushes every singular value of the update towards 1, so the 1e-3 relative difference between a
    # gradient summed over two ranks and one summed over the whole batch moves a Muon update by percents per
    # step (measured 5.7e-2 after four steps); AdamW updates follow their gradients.
    assert relative(results[0][1] - weights, whole_weights - weights) < (1e-1 if mode == "muon" else 5e-2)
    if mode == "fp32":  # tensor by tensor: a wrongly scaled small bucket (norm scales, biases) cannot hide
        for offset, rows, cols in bridge.parameter_layout(single):
            part = slice(offset, offset + rows * max(cols, 1))
            moved = whole_weights[part] - weights[part]
            if np.abs(moved).max() > 0:
                assert relative(results[0][1][part] - weights[part], moved) < 1e-4, (offset, rows, cols)
        np.testing.assert_allclose(results[0][0], whole_losses, rtol=1e-5, atol=1e-5)
