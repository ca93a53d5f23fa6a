"""The CPU oracle against fixtures generated from the reference itself (tests/golden/make_golden.py)."""
import json

import numpy as np
import pytest
import torch

from oracle import indexing
from oracle.model import Arch, Model, parameter_count, specification
from oracle.optim import Hyper, OneCycle, Optimizer, onecycle_point
from helpers import relative


@pytest.mark.parametrize("depth,context", [(4, 4), (8, 8), (4, 8)])
def test_model_matches_reference_model(golden, depth, context):
    torch.set_num_threads(1)
    g = np.load(golden / f"model_d{depth}_c{context}.npz")
    model = Model(Arch.reference(depth))
    model.load(g["weights"])
    logits, grad, losses = model.batch(g["x"], g["y"])
    # Same operations in the same order as tests/reference.py: equal up to summation order.
    np.testing.assert_allclose(logits, g["logits"], rtol=0, atol=1e-6)
    assert relative(grad, g["gradient"]) < 1e-6
    np.testing.assert_allclose(losses, g["losses"], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name,scheduled", [("optimizer", False), ("optimizer_onecycle", True)])
def test_optimizer_matches_torch(golden, name, scheduled):
    """tests/verify.py:64-105 with the oracle in the engine's place."""
    g = np.load(golden / f"{name}.npz")
    opt = Optimizer(Arch.reference(4), Hyper(clip=0), g["initial"], schedule=OneCycle(20) if scheduled else None)
    rng = np.random.default_rng(192)
    for _ in range(20):
        opt.step((rng.standard_normal(len(g["initial"])) * .01).astype(np.float32))
    a = g["adam_mask"]
    assert relative(opt.w - g["initial"], g["expected"] - g["initial"]) < .04
    assert relative(opt.w[a] - g["initial"][a], g["expected"][a] - g["initial"][a]) < 1e-4
    np.testing.assert_allclose(opt.w[a], g["expected"][a], atol=2e-6, rtol=2e-5)


def test_small_updates_retained(golden):
    """tests/verify.py:108-127: FP32 masters keep updates below one BF16 ulp."""
    expected = np.load(golden / "small_updates.npz")["expected"]
    arch = Arch.reference(4)
    n = parameter_count(arch)
    opt = Optimizer(arch, Hyper(learning_rate=1e-5, weight_decay=0, clip=0), np.full(n, .5, np.float32))
    for _ in range(64):
        opt.step(np.full(n, .01, np.float32))
    mask = np.concatenate([np.full(int(np.prod(s)), not (len(s) == 2 and name.split(".")[-1] not in ("embedding", "head")))
                           for name, s in specification(arch)])
    np.testing.assert_allclose(opt.w[mask], expected[0], atol=2e-6, rtol=0)
    assert np.max(np.abs(opt.w[mask] - .5)) > .0005


def test_hash_and_onecycle_known_answers(golden):
    h = json.loads((golden / "ref_host.json").read_text())
    lib = indexing.load()
    for key, value in h["hash_u64"]:
        assert indexing.hash_u64(int(key)) == int(value)
        assert lib.oracle_hash_u64(int(key)) == int(value)
    for total, step, multiplier, momentum in h["onecycle"]:
        m, mo = onecycle_point(OneCycle(total), step)
        assert m.view(np.uint32) == multiplier and mo.view(np.uint32) == momentum
    for total, step, lr, momentum in json.loads((golden / "onecycle_torch.json").read_text()):
        m, mo = onecycle_point(OneCycle(total), step)
        np.testing.assert_allclose(m, lr, rtol=1e-7, atol=1e-12)
        np.testing.assert_allclose(mo, momentum, rtol=1e-7, atol=1e-8)
    assert parameter_count(Arch.reference(4)) == h["parameter_count"]["4"]
    assert parameter_count(Arch.reference(8)) == h["parameter_count"]["8"]


def test_byte_batches_c_and_python_agree():
    data = np.random.default_rng(718).integers(0, 256, 4096, dtype=np.uint8)
    for context, batch, world in [(4, 16, 1), (8, 5, 1), (256, 3, 1), (8, 4, 2)]:
        for rank in range(world):
            for step in (0, 1, 12345):
                a = indexing.byte_batch(data, 3407, step, batch, context, world, rank)
                b = indexing.byte_batch_c(data, 3407, step, batch, context, world, rank)
                np.testing.assert_array_equal(a[0], b[0])
                np.testing.assert_array_equal(a[1], b[1])
                np.testing.assert_array_equal(a[0][:, 1:], a[1][:, :-1])  # y is x shifted by one byte
    # The reference's own statement of the rule (tests/pipeline.py:75-78) for ctx <= 8.
    e = 8 + indexing.hash_u64(3407 + 5 * 16 + 3) % (4096 - 8)
    assert indexing.endpoint(3407, 5, 16, 3, 4, 4096) == e


def test_data_parallel_shards_tile_the_global_batch():
    """World-W ranks draw exactly the sequences one engine with batch W*B would draw."""
    data = np.random.default_rng(5).integers(0, 256, 8192, dtype=np.uint8)
    whole = indexing.byte_batch(data, 7, 9, 12, 8)
    parts = [indexing.byte_batch(data, 7, 9, 4, 8, world=3, rank=r) for r in range(3)]
    np.testing.assert_array_equal(np.concatenate([p[0] for p in parts]), whole[0])
    np.testing.assert_array_equal(np.concatenate([p[1] for p in parts]), whole[1])


def test_gpt_architecture_oracle_is_consistent():
    """BF16-rounded and FP32 variants of the scaled architecture agree to BF16 precision, and
    the parameter count is the one the benchmark's FLOP model uses."""
    assert parameter_count(Arch.gpt(12, 768, 12)) == 85169664
    arch = Arch.gpt(2, 64, 2)
    rng = np.random.default_rng(0)
    x = rng.integers(0, 256, (2, 16), dtype=np.uint8)
    y = rng.integers(0, 256, (2, 16), dtype=np.uint8)
    a, b = Model(arch, seed=1), Model(arch, seed=1, fp32=True)
    la, ga, _ = a.batch(x, y)
    lb, gb, _ = b.batch(x, y)
    assert relative(la, lb) < 2e-2 and relative(ga, gb) < 5e-2
