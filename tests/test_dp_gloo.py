"""Host-side logic of data parallelism on CPU ranks (gloo, world size 2): rank-sharded byte
sampling tiles the global batch, and summing per-rank gradients of loss/(global count) gives the
single-engine gradient of the global batch — the contract the NCCL path of the engine implements."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import indexing
from oracle.model import Arch, Model


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    batch, context, step, seed = 4, 8, 5, 3407
    data = np.random.default_rng(9).integers(0, 256, 4096, dtype=np.uint8)
    model = Model(Arch.reference(4), scale=.08)
    x, y = indexing.byte_batch(data, seed, step, batch, context, world=world, rank=rank)
    _, grad, losses = model.batch(x, y, divisor=world * batch * context)
    g = torch.from_numpy(grad)
    dist.all_reduce(g)                      # the engine's gradient exchange: a sum over ranks
    l = torch.from_numpy(losses.copy())
    dist.all_reduce(l)                      # per-position means: mean over ranks
    gathered = [torch.zeros(batch, context, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(x))
    if rank == 0:
        wx, wy = indexing.byte_batch(data, seed, step, world * batch, context)
        _, whole_grad, whole_losses = model.batch(wx, wy)
        out.put((np.array_equal(torch.cat(gathered).numpy(), wx),
                 float(np.abs(g.numpy() - whole_grad).max() / np.abs(whole_grad).max()),
                 float(np.abs(l.numpy() / world - whole_losses).max())))
    dist.destroy_process_group()


def test_two_rank_gradient_sum_equals_global_batch():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    same_bytes, grad_error, loss_error = out.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert same_bytes
    assert grad_error < 2e-2   # BF16 gradient roundings differ between a 4- and an 8-sequence batch
    assert loss_error < 1e-6
