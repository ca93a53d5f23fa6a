"""Failure detection without a GPU fault.

CPU: configurations that do not agree among the ranks of a data-parallel job are refused before any
engine or communicator exists (gloo, world size 2), and bad configurations are refused by
tg_create_ex before the device is touched.
GPU: a device-side wait that runs out (a barrier nothing arms, ~1 ms limit, nothing in flight)
leaves an error code that the next synchronising call reports; the engine stays usable."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from turbogpt_b200 import Config, ConfigEx, Native, bridge


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, case, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hidden = 512 if (case == "hidden" and rank == 1) else 256
    claimed_world = 3 if (case == "world" and rank == 1) else world
    claimed_rank = 0 if case == "rank" else rank
    ex = ConfigEx.gpt(Config(depth=2, context=64, batch=4), 128, 2, hidden, world=claimed_world, rank=claimed_rank,
                      flags=bridge.FLAG_NO_COMMUNICATOR)

    def all_gather(value):
        gathered = [None] * world
        dist.all_gather_object(gathered, value)
        return gathered

    try:
        bridge.require_matching_ranks(ex, all_gather)
        out.put((rank, "accepted"))
    except RuntimeError as error:
        out.put((rank, str(error)))
    dist.destroy_process_group()


@pytest.mark.parametrize("case", ["same", "hidden", "world", "rank"])
def test_mismatched_ranks_are_refused_before_any_engine_exists(case):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, case, out)) for r in range(2)]
    for p in procs:
        p.start()
    answers = dict(out.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    if case == "same":
        assert answers == {0: "accepted", 1: "accepted"}
    else:
        assert all("data-parallel job" in a for a in answers.values()), answers


def test_bad_configurations_are_refused_without_a_device():
    lib = bridge.load_library()
    ex = ConfigEx.gpt(Config(depth=2, context=64, batch=4), 128, 2)
    assert lib.tg_ex_config_digest(C.byref(ex)) != 0
    other = ConfigEx.gpt(Config(depth=2, context=64, batch=4, device=3), 128, 2, rank=0)
    assert lib.tg_ex_config_digest(C.byref(other)) == lib.tg_ex_config_digest(C.byref(ex))
    for change, message in [(dict(struct_size=100), b"struct_size"), (dict(world=2, rank=2), b"rank"),
                            (dict(world=0), b"world"), (dict(width=100), b"width")]:
        bad = ConfigEx.gpt(Config(depth=2, context=64, batch=4), 128, 2)
        for key, value in change.items():
            setattr(bad, key, value)
        assert lib.tg_ex_config_digest(C.byref(bad)) == 0
        assert not lib.tg_create_ex(C.byref(bad))
        assert message in lib.tg_error(), (change, lib.tg_error())


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_the_engine_survives():
    rng = np.random.default_rng(0)
    x = rng.integers(0, 256, (4, 64), dtype=np.uint8)
    ex = ConfigEx.gpt(Config(depth=1, context=64, batch=4, clip=0), 128, 2)
    with Native(ex) as engine:
        weights = bridge.initialize_weights(ex)
        engine.set_weights(weights)
        before, _, _ = engine.batch(x, x, backward=False)
        assert engine.lib.tg_ex_selftest_bounded_wait(engine.handle, 1.0) == 1   # gave up, as designed
        logits = np.empty((4, 64, 256), np.float32)
        losses = np.empty(64, np.float32)
        status = engine.lib.tg_batch(engine.handle, x.ctypes.data, x.ctypes.data, logits.ctypes.data, None,
                                     losses.ctypes.data)
        assert status < 0 and b"wait gave up (code 901)" in engine.lib.tg_error()
        engine.set_weights(weights)                                              # clears the error word
        after, _, _ = engine.batch(x, x, backward=False)
        np.testing.assert_array_equal(before, after)
        assert engine.lib.tg_ex_selftest_bounded_wait(engine.handle, 0.0) < 0    # limit out of range
