"""Generates the committed fixtures in this directory from the reference itself.

Runs only in the development container, where the reference tree is mounted; the
tests read the fixtures, never the reference.  Usage:

    python tests/golden/make_golden.py /path/to/reference

* ref_host.json        — known answers printed by ref_probe.cpp, which includes the
                         reference's host headers (hash_u64, parameter layout, OneCycle
                         points, struct sizes, initial weights checksum).
* model_d{D}_c{T}.npz  — tests/reference.py (imported unmodified, device='cpu') on the
                         fixture of tests/verify.py:14-33: weights Reference(seed 42,
                         scale .08), bytes default_rng(71); logits, gradient of the mean
                         loss, per-position loss.
* optimizer*.npz       — tests/verify.py:64-105: 20 injected-gradient steps of
                         torch.optim.AdamW + torch.optim.Muon, without and with OneCycleLR.
* small_updates.npz    — tests/verify.py:108-127.
* onecycle_torch.json  — tests/verify.py:177-200: torch OneCycleLR multipliers/momenta.
"""
import json
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch
from torch.nn import functional as F

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]


def main(reference_root: str):
    root = Path(reference_root)
    sys.path.insert(0, str(root / "tests"))
    from reference import Reference  # the reference's own numerical model

    out = REPO / "oracle" / "_ref"
    out.mkdir(parents=True, exist_ok=True)
    exe = out / "ref_probe"
    subprocess.check_call(["g++", "-O1", "-std=c++17", f"-I{root}", str(HERE / "ref_probe.cpp"),
                           str(root / "model.cpp"), "-o", str(exe)])
    (HERE / "ref_host.json").write_text(subprocess.check_output([str(exe)]).decode())

    torch.set_num_threads(1)  # fixed summation order
    for depth, context, batch in [(4, 4, 16), (8, 8, 16), (4, 8, 12)]:
        cfg = SimpleNamespace(depth=depth, context=context, batch=batch)
        ref = Reference(cfg, device="cpu", seed=42, scale=.08)
        rng = np.random.default_rng(71)
        x = rng.integers(0, 256, (batch, context), dtype=np.uint8)
        y = rng.integers(0, 256, x.shape, dtype=np.uint8)
        logits = ref.forward(torch.tensor(x).long())
        loss = F.cross_entropy(logits.flatten(0, 1), torch.tensor(y).long().flatten(),
                               reduction="none").reshape(x.shape)
        loss.mean().backward()
        grad = torch.cat([p.grad.flatten() for p in ref.params.values()]).numpy()
        np.savez_compressed(HERE / f"model_d{depth}_c{context}.npz", weights=ref.flat(), x=x, y=y,
                            logits=logits.detach().numpy().astype(np.float32), gradient=grad,
                            losses=loss.detach().mean(0).numpy())

    def hidden_matrix(name, p):
        return p.ndim == 2 and name not in ("embedding", "head")

    hyper = dict(learning_rate=.0006, muon_lr=.02, beta1=.9, beta2=.95, momentum=.95,
                 weight_decay=.1, epsilon=1e-8, ns_steps=5)
    for scheduled in (False, True):
        cfg = SimpleNamespace(depth=4, context=4, batch=4)
        ref = Reference(cfg, device="cpu")
        initial = ref.flat()
        groups, matrices = [], []
        for name, p in ref.params.items():
            if hidden_matrix(name, p):
                matrices.append(p)
            else:
                groups.append({"params": [p], "weight_decay": hyper["weight_decay"] if name == "head" else 0})
        adam = torch.optim.AdamW(groups, lr=hyper["learning_rate"], betas=(hyper["beta1"], hyper["beta2"]),
                                 eps=hyper["epsilon"], foreach=False, fused=False)
        muon = torch.optim.Muon(matrices, lr=hyper["muon_lr"], momentum=hyper["momentum"],
                                weight_decay=hyper["weight_decay"], ns_steps=hyper["ns_steps"])
        schedulers = []
        if scheduled:
            schedulers.append(torch.optim.lr_scheduler.OneCycleLR(adam, max_lr=hyper["learning_rate"], total_steps=20))
            schedulers.append(torch.optim.lr_scheduler.OneCycleLR(muon, max_lr=hyper["muon_lr"], total_steps=20))
        rng = np.random.default_rng(192)
        count = len(initial)
        for _ in range(20):
            grad = (rng.standard_normal(count) * .01).astype(np.float32)
            offset = 0
            for p in ref.params.values():
                p.grad = torch.tensor(grad[offset:offset + p.numel()].reshape(p.shape))
                offset += p.numel()
            adam.step()
            muon.step()
            for s in schedulers:
                s.step()
        mask = np.concatenate([np.full(p.numel(), not hidden_matrix(n, p)) for n, p in ref.params.items()])
        np.savez_compressed(HERE / f"optimizer{'_onecycle' if scheduled else ''}.npz", initial=initial,
                            expected=ref.flat(), adam_mask=mask)

    # Sub-BF16-ULP retention (verify.py:108-127): 64 AdamW steps of lr 1e-5 on w = .5, g = .01.
    p = torch.nn.Parameter(torch.full((64,), .5))
    opt = torch.optim.AdamW([p], lr=1e-5, betas=(.9, .95), eps=1e-8, weight_decay=0, foreach=False)
    for _ in range(64):
        p.grad = torch.full((64,), .01)
        opt.step()
    np.savez_compressed(HERE / "small_updates.npz", expected=p.detach().numpy())

    points = []
    for total in (8, 20, 37, 48829, 488282):
        param = torch.nn.Parameter(torch.ones(1))
        optimizer = torch.optim.AdamW([param], lr=.0006)
        sched = torch.optim.lr_scheduler.OneCycleLR(optimizer, max_lr=.0006, total_steps=total)
        steps = range(total) if total < 100 else sorted(set(
            [0, 1, total - 2, total - 1] + [int(.3 * total) + j for j in (-2, -1, 0, 1)] +
            [int(total * f) for f in (.1, .5, .9)]))
        for step in steps:
            sched.last_epoch = step
            lr = sched.get_lr()[0] / .0006
            points.append([total, step, float(lr), float(optimizer.param_groups[0]["betas"][0])])
    (HERE / "onecycle_torch.json").write_text(json.dumps(points))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
