"""The data-parallel training host (turbogpt_b200/turbogpt_dp, host/train_dp.cpp): argument and
configuration errors on CPU; on a GPU a short run, its log and checkpoint, and that a run stopped
half way and resumed with --load ends with bit-identical weights — on one device and, where the box
has them, on two (NCCL inside the engines, one thread per device)."""
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from turbogpt_b200.build import HOST, build_host

MODEL = ["--depth", "2", "--width", "128", "--heads", "2", "--hidden", "256", "--context", "64", "--batch", "4"]


def _host():
    if not HOST.exists():
        build_host()
    return str(HOST)


def _corpus(tmp_path):
    path = tmp_path / "corpus.bin"
    path.write_bytes(np.random.default_rng(4).integers(0, 48, 1 << 15, dtype=np.uint8).tobytes())
    return str(path)


def test_argument_errors(tmp_path):
    host = _host()
    assert subprocess.run([host], capture_output=True).returncode == 2
    assert subprocess.run([host, "--data", "x", "--log-to", str(tmp_path), "--optimizer", "sgd"],
                          capture_output=True).returncode == 2
    missing = subprocess.run([host, "--data", str(tmp_path / "none"), "--log-to", str(tmp_path)], capture_output=True,
                             text=True)
    assert missing.returncode == 1 and "Cannot open" in missing.stderr
    bad = subprocess.run([host, "--data", _corpus(tmp_path), "--log-to", str(tmp_path), "--width", "100"],
                         capture_output=True, text=True)
    assert bad.returncode == 1 and "width" in bad.stderr


def _run(tmp_path, name, devices, extra):
    out = tmp_path / name
    command = [_host(), "--data", _corpus(tmp_path), "--log-to", str(out), "--devices", devices, "--tokens",
               str(8 * 4 * 64 * len(devices.split(","))), "--chunk", "2", *MODEL, *extra]
    done = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr + done.stdout
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("devices,optimizer", [("0", "adamw"), ("0", "muon"), ("0,1", "adamw"), ("0,1", "muon")])
def test_stopped_and_resumed_run_equals_uninterrupted_run(tmp_path, devices, optimizer):
    if len(devices.split(",")) > torch.cuda.device_count():
        pytest.skip("needs two GPUs")
    whole = _run(tmp_path, "whole", devices, ["--optimizer", optimizer])
    log = (whole / "train.log").read_text().splitlines()
    steps = [line for line in log if line.startswith("step ")]
    assert len(steps) == 4 and steps[-1].startswith("step 8 ") and "checkpoint at step 8" in log[-1]
    losses = [float(line.split()[3]) for line in steps]
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]
    first = _run(tmp_path, "parts", devices, ["--optimizer", optimizer, "--stop-after", "4"])
    assert "checkpoint at step 4" in (first / "train.log").read_text()
    _run(tmp_path, "parts", devices, ["--optimizer", optimizer, "--load", str(first / "model.pt")])
    a = torch.load(whole / "model.pt", weights_only=True)
    b = torch.load(first / "model.pt", weights_only=True)
    assert int(a["opt"]["step"]) == int(b["opt"]["step"]) == 8
    for group, key in [("model", "weights"), ("opt", "momentum"), ("opt", "variance")]:
        assert torch.equal(a[group][key], b[group][key]), key
    assert a["model"]["architecture"].tolist()[:3] == [128, 2, 256]
    refused = subprocess.run([_host(), "--data", _corpus(tmp_path), "--log-to", str(first), "--devices", devices,
                              "--tokens", str(8 * 4 * 64 * len(devices.split(","))), *MODEL, "--optimizer", optimizer,
                              "--load", str(first / "model.pt")], capture_output=True, text=True)
    assert refused.returncode == 1 and "already reached" in refused.stderr
