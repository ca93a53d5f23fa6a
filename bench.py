"""Benchmark of the dense training step (tokens/s and MFU) on N B200s of one node.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --workload config5 ...    # the larger, longer-context step (Muon + AdamW)
    python bench.py --impl reference ...      # the CPU arm: the oracle port on the host cores

Default workload ("config3"): 12 layers, d_model 768, 12 heads, MLP 3072, vocab 256, context 1024,
micro-batch 32 per GPU, BF16 compute with FP32 masters, AdamW with global-norm clipping.
"config5": 16 layers, d_model 1024, 16 heads, MLP 4096, context 4096, micro-batch 8 per GPU, Muon
(5 Newton-Schulz iterations) on the 2-D hidden matrices and AdamW on embedding and norms.
Synthetic bytes from a seeded order-2 Markov chain whose 65 536 transition rows are Dirichlet(0.1).
A step is sampling, forward, loss, backward, gradient all-reduce in BF16 buckets (N > 1),
optimizer.  Rank 0 prints one JSON line.  With N > 1 the line also carries `dp_check`: after the
timed region the replicas' weights must be bit-identical, and the first step's loss must equal what
one engine computes on the same global batch.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
WORKLOADS = {
    "config3": dict(depth=12, width=768, heads=12, hidden=3072, context=1024, batch=32, optimizer="adamw",
                    name="gpt-12L-768d-12h-ctx1024-mb32-adamw-markov2-bytes"),
    "config5": dict(depth=16, width=1024, heads=16, hidden=4096, context=4096, batch=8, optimizer="muon",
                    name="gpt-16L-1024d-16h-ctx4096-mb8-muon5-adamw-markov2-bytes"),
}
TRAFFIC_SUMMARY = ROOT / "profiles" / "gemm_tc_forward_32768x3072x768.md"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def markov_bytes(size: int, seed: int = 0) -> np.ndarray:
    """Order-2 Markov chain over bytes; each of the 65 536 transition rows ~ Dirichlet(0.1).
    Many chains advance in lock-step (vectorised) and are concatenated."""
    rng = np.random.default_rng(seed)
    table = rng.gamma(0.1, size=(65536, 256)).astype(np.float32) + 1e-30
    cdf = np.cumsum(table / table.sum(1, keepdims=True), axis=1)
    cdf[:, -1] = 1.0
    chains = 2048
    length = (size + chains - 1) // chains
    out = np.empty((chains, length), np.uint8)
    a = rng.integers(0, 256, chains)
    b = rng.integers(0, 256, chains)
    stream = np.random.default_rng(seed + 1)
    for t in range(length):
        u = stream.random(chains, dtype=np.float32)
        nxt = (cdf[a * 256 + b] < u[:, None]).sum(1).clip(0, 255)
        out[:, t] = nxt
        a, b = b, nxt
    return out.reshape(-1)[:size].copy()


def flops_per_token(w) -> dict:
    W, Hd, L, T = w["width"], w["hidden"], w["depth"], w["context"]
    matrix_params = L * (3 * W * W + W * W + 2 * Hd * W) + 256 * W
    gemm = 2 * matrix_params                   # one pass over every matrix
    attention_forward = 4 * T * W * L / 2      # QK^T and PV, causal half
    return {"gemm_pass": gemm, "attention_forward": attention_forward,
            "total": 3 * gemm + 3.5 * attention_forward}   # = 6 N + 6 L T d + recomputed scores in backward


def model_flops_per_token(w) -> float:
    """The conventional count used for MFU: 6 x matrix parameters + causal attention 6 L T d."""
    W, Hd, L, T = w["width"], w["hidden"], w["depth"], w["context"]
    return 6.0 * (L * (3 * W * W + W * W + 2 * Hd * W) + 256 * W) + 6.0 * L * T * W


def captured_traffic() -> tuple[float | None, str]:
    """DRAM bytes (read + write) of one launch of the step's largest GEMM, as recorded in the ncu
    summary under profiles/ (the line `dram_bytes_per_launch: <number>`): a figure from that capture,
    not something this run measures."""
    import re
    if TRAFFIC_SUMMARY.exists():
        found = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)", TRAFFIC_SUMMARY.read_text())
        if found:
            return float(found.group(1)), f"ncu capture summarised in profiles/{TRAFFIC_SUMMARY.name}"
    return None, "no ncu summary found"


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return FALLBACK_PEAKS, "fallback"


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(device)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        self.process.wait()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().strip().splitlines() if r.strip()]
        os.unlink(self.file.name)
        clocks, reasons, max_clock = [], set(), None
        for r in rows:
            try:
                clocks.append(float(r[1]))
                max_clock = float(r[2])
            except (ValueError, IndexError):
                continue
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for name, value in zip(names, r[5:9]):
                if value.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def cpu_step_tokens_per_second(w: dict, batch: int, steps: int = 1) -> tuple[float, int, str]:
    """The oracle port (oracle/model.py + oracle/optim.py) doing forward + backward + the workload's
    optimizer on the host cores, on `batch` sequences of the workload's context."""
    import torch
    from oracle.model import Arch, Model
    from oracle.optim import Hyper, Optimizer
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    arch = Arch.gpt(w["depth"], w["width"], w["heads"], w["hidden"])
    model = Model(arch, seed=1)
    opt = Optimizer(arch, Hyper(learning_rate=3e-4, clip=1.0), model.flat(), hidden=w["optimizer"])
    rng = np.random.default_rng(0)
    data = rng.integers(0, 256, batch * w["context"] + 1, dtype=np.uint8)
    x = data[:-1].reshape(batch, w["context"])
    y = data[1:].reshape(batch, w["context"])
    times = []
    for _ in range(steps):
        start = time.perf_counter()
        model.load(opt.w)
        _, grad, _ = model.batch(x, y)
        opt.step(grad)
        times.append(time.perf_counter() - start)
    seconds = float(np.mean(times))
    return (batch * w["context"] / seconds, cores,
            f"{batch} x {w['context']} tokens per step, {steps} step(s), fwd+bwd+{w['optimizer']}")


def reference_arm(args, w: dict) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(min(args.warmup, 1)):
        cpu_step_tokens_per_second(w, 1, 1)
    start = time.perf_counter()
    value, cores, sample = cpu_step_tokens_per_second(w, 1, max(1, args.steps))
    elapsed = time.perf_counter() - start
    print(json.dumps({
        "impl": "reference", "metric": "train_tokens_per_second", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000 * elapsed / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "note": "CPU port of the reference's numerical model (tests/reference.py "
                   "generalised); each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200")
    parser.add_argument("--workload", default="config3", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-roofline", action="store_true")
    parser.add_argument("--fp32-exchange", action="store_true", help="all-reduce FP32 gradient buckets instead of BF16")
    parser.add_argument("--flags", type=int, default=0, help="extra TgConfigEx flags (debugging)")
    args = parser.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        reference_arm(args, w)
        return

    import ctypes as C
    import torch
    from turbogpt_b200 import Config, ConfigEx, Native, bridge

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    lib = bridge.load_library()
    muon = w["optimizer"] == "muon"
    flags = args.flags
    if world > 1 and not args.fp32_exchange:
        flags |= bridge.FLAG_BF16_GRADIENT_EXCHANGE

    def configuration(**changes):
        base = Config(depth=w["depth"], context=w["context"], batch=w["batch"], device=local, learning_rate=3e-4,
                      beta1=.9, beta2=.95, weight_decay=.1, clip=1.0, seed=3407, ns_steps=5)
        return ConfigEx.gpt(base, w["width"], w["heads"], w["hidden"],
                            hidden_optimizer=bridge.HIDDEN_MUON if muon else bridge.HIDDEN_ADAMW, **changes)

    ex = configuration(world=world, rank=rank, flags=flags)
    if world > 1:
        import torch.distributed as dist
        backend = os.environ.get("BENCH_DIST_BACKEND", "nccl")
        dist.init_process_group(backend)
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda" if backend == "nccl" else "cpu")
        if rank == 0:
            host = np.zeros(128, np.uint8)
            if lib.tg_ex_nccl_unique_id(host.ctypes.data) < 0:
                raise SystemExit(lib.tg_error().decode())
            ident.copy_(torch.from_numpy(host))
        dist.broadcast(ident, 0)
        ident_host = np.ascontiguousarray(ident.cpu().numpy())  # keep alive across the copy
        C.memmove(ex.nccl_id, ident_host.ctypes.data, 128)

        def all_gather(value):
            gathered = [None] * world
            dist.all_gather_object(gathered, value)
            return gathered

        bridge.require_matching_ranks(ex, all_gather)  # before any engine or communicator exists

    data = markov_bytes(8 << 20, seed=0)
    initial = bridge.initialize_weights(ex)
    engine = Native(ex)
    engine.set_weights(initial)
    engine.set_data(data)
    stream = torch.cuda.ExternalStream(lib.tg_ex_stream(engine.handle), device=local)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 1)
    first_x, first_y = engine.sample(0)  # this rank's bytes of step 0, for the data-parallel check
    engine.train(warmup)
    first_loss = float(engine.training_losses(1).mean())
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches_before = lib.tg_ex_launch_count(engine.handle)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    engine.train(args.steps)
    end.record(stream)
    barrier()
    milliseconds = begin.elapsed_time(end)
    launches = lib.tg_ex_launch_count(engine.handle) - launches_before
    clocks = sampler.stop() if sampler else None
    last_loss = float(engine.training_losses(args.steps)[-1].mean())
    if world > 1:
        t = torch.tensor([milliseconds], device=ident.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        milliseconds = float(t.item())
    tokens_per_step = w["batch"] * w["context"] * world
    value = tokens_per_step * args.steps / (milliseconds / 1000)

    # End to end through the host-buffer API: every step copies that step's bytes from pinned
    # host memory, trains on them and reads the per-position losses back.
    rng = np.random.default_rng(rank)
    pinned_x = torch.empty(w["batch"], w["context"], dtype=torch.uint8).pin_memory()
    pinned_y = torch.empty_like(pinned_x).pin_memory()
    hx, hy = pinned_x.numpy(), pinned_y.numpy()
    e2e_steps = max(2, min(args.steps, 10))
    barrier()
    start = time.perf_counter()
    for _ in range(e2e_steps):
        ends = rng.integers(w["context"], len(data) - 1, w["batch"])
        for i, e in enumerate(ends):
            hx[i] = data[e - w["context"]:e]
            hy[i] = data[e - w["context"] + 1:e + 1]
        engine.train_batch(hx, hy, want_losses=True)
    barrier()
    e2e_seconds = time.perf_counter() - start
    if world > 1:
        t = torch.tensor([e2e_seconds], device=ident.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    e2e_value = tokens_per_step * e2e_steps / e2e_seconds
    memory_gb = engine.memory_gb()

    dp_check = None
    if world > 1:
        # (1) Replicas must hold bit-identical weights after all those steps (each rank trained on its
        # own bytes; only the summed gradients are shared).  (2) The first step's loss of the
        # data-parallel job must be what ONE engine computes on the same global batch: every rank's
        # step-0 bytes go to rank 0, which evaluates them with the initial weights.
        final = engine.weights()
        digest = int(np.bitwise_xor.reduce(final.view(np.uint32).astype(np.uint64) * np.arange(1, final.size + 1, dtype=np.uint64)))
        low = torch.tensor([digest >> 32, digest & 0xffffffff], device=ident.device, dtype=torch.float64)
        high = low.clone()
        dist.all_reduce(low, op=dist.ReduceOp.MIN)
        dist.all_reduce(high, op=dist.ReduceOp.MAX)
        replicas_identical = bool(torch.equal(low, high))
        gathered = [None] * world
        dist.all_gather_object(gathered, (first_x, first_y))
        single_loss = None
        if rank == 0:
            single = Native(configuration())
            single.set_weights(initial)
            losses = [single.batch(x, y, backward=False)[2].mean() for x, y in gathered]
            single.close()
            single_loss = float(np.mean(losses))
        dp_check = {"replicas_identical": replicas_identical, "first_step_loss": first_loss,
                    "single_engine_loss_on_global_batch": single_loss,
                    "loss_agrees_2e-3": single_loss is not None and abs(single_loss - first_loss) <= 2e-3,
                    "exchange": "fp32" if args.fp32_exchange else "bf16"}
    engine.close()

    peak, peak_source = peaks()
    mfu_flops = model_flops_per_token(w)
    result = {
        "metric": "train_tokens_per_second", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": milliseconds / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "global_batch": w["batch"] * world, "seq_len": w["context"],
                   "parallelism": f"dp{world}", "l2": "per-step working set (>10 GB of activations) exceeds the 126 MB L2",
                   "data_detail": "order-2 Markov bytes, Dirichlet(0.1) rows, seed 0, 8 MiB"},
        "tokens_per_second_per_gpu": value / world,
        "mfu_nominal_2250": mfu_flops * value / world / 2.25e15,
        "mfu_of_measured_sustained": mfu_flops * value / world / (peak["bf16_tflops_sustained"] * 1e12),
        "model_flops_per_token": mfu_flops, "loss_first": first_loss, "loss_last": last_loss,
        "memory_gb": memory_gb, "clocks": clocks, "gpu_launches": int(launches),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * w["batch"] * w["context"] * world,
                "d2h_bytes_per_step": 4 * w["context"] * world, "steps": e2e_steps,
                "api": "tg_ex_train_batch (host bytes in, per-position losses out, every step)"},
    }
    if dp_check is not None:
        result["dp_check"] = dp_check

    if rank == 0 and not args.no_roofline:
        # Per-family device time from a profiled engine (CUDA events around every launch on the
        # engine's stream, no graph replay), a few steps right after the timed region, with the SM
        # clock sampled over those steps so that clock and schedule effects can be told apart.
        profiled = Native(configuration(flags=args.flags | bridge.FLAG_PROFILE))
        profiled.set_weights(initial)
        profiled.set_data(data)
        profiled.train(1)
        profiled.training_losses(1)
        profiled.profile(reset=True)
        steps = 3 if w is WORKLOADS["config3"] else 2
        profile_clocks = ClockSampler(local)
        profiled.train(steps)
        profiled.training_losses(steps)
        profile_clocks = profile_clocks.stop()
        families = profiled.profile()
        profiled.close()
        per_step = {k: {"ms": v[0] / steps, "launches": v[1] // steps} for k, v in families.items() if v[1]}
        f = flops_per_token(w)
        tokens = w["batch"] * w["context"]
        work = {"gemm_forward": f["gemm_pass"] * tokens, "gemm_input_grad": f["gemm_pass"] * tokens,
                "gemm_weight_grad": f["gemm_pass"] * tokens, "attention_forward": f["attention_forward"] * tokens,
                "attention_backward": 2.5 * f["attention_forward"] * tokens}
        # the profiled leg is short: with too few samples of its own it borrows the timed region's median clock
        if (profile_clocks.get("samples") or 0) < 4 and clocks and clocks.get("sm_mhz"):
            profile_clocks = dict(profile_clocks, sm_mhz=clocks["sm_mhz"], borrowed_from="the timed region")
        mhz = profile_clocks.get("sm_mhz")
        for k, flop in work.items():
            if k in per_step and per_step[k]["ms"] > 0:
                per_step[k]["tflops"] = flop / (per_step[k]["ms"] * 1e-3) / 1e12
                if mhz:  # the same work per SM clock: FLOP per cycle per SM (dense BF16 peak is 8192)
                    per_step[k]["flop_per_clock_per_sm"] = flop / (per_step[k]["ms"] * 1e-3 * mhz * 1e6 * 148)
        # The dominant kernel is gemm_tc_kernel: every projection, input-gradient and weight-gradient
        # GEMM of the step (three passes over the parameters), timed live above.
        gemm_families = [k for k in ("gemm_forward", "gemm_input_grad", "gemm_weight_grad") if k in per_step]
        gemm_seconds = sum(per_step[k]["ms"] * 1e-3 for k in gemm_families)
        gemm_launches = sum(per_step[k]["launches"] for k in gemm_families)
        achieved = sum(work[k] for k in gemm_families) / gemm_seconds / 1e12
        tensor_families = [k for k in work if k in per_step]
        all_tensor = sum(work[k] for k in tensor_families) / sum(per_step[k]["ms"] * 1e-3 for k in tensor_families) / 1e12
        traffic, traffic_source = captured_traffic()
        result["roofline"] = {
            "bound": "tensor", "achieved": achieved, "peak": peak["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": achieved / peak["bf16_tflops_sustained"], "peak_source": peak_source,
            "kernel": "gemm_tc_kernel (all GEMMs of the step)", "launches_per_step": gemm_launches,
            "flop_per_launch": sum(work[k] for k in gemm_families) / max(gemm_launches, 1),
            "us_per_launch": gemm_seconds * 1e6 / max(gemm_launches, 1),
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the largest GEMM shape of
            # config 3 (32768 x 3072 x 768, algorithmic 256 MB): read from the committed ncu summary,
            # not measured by this run
            "traffic": traffic, "traffic_shape": "32768x3072x768 up-projection", "traffic_source": traffic_source,
            "share_of_step": gemm_seconds * 1e3 / sum(v["ms"] for v in per_step.values()),
            "all_tensor_families": {"achieved": all_tensor, "frac": all_tensor / peak["bf16_tflops_sustained"],
                                    "note": "GEMMs + attention forward/backward, causal FLOP count"},
            "profiled_steps_clocks": profile_clocks,
            "families_ms_per_step": per_step,
        }
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        cpu_step_tokens_per_second(w, 1, 1)  # warm-up: thread pools, allocations
        cpu_value, cores, sample = cpu_step_tokens_per_second(w, 4, 2)  # about 15-25 s of host work
        result["cpu_baseline"] = {"value": cpu_value, "unit": "tokens/s", "cores": cores, "kind": "port",
                                  "sample": sample}
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.path.insert(0, str(ROOT))
    main()
