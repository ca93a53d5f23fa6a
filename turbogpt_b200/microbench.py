"""Kernel microbenchmarks through the C ABI (device-resident BF16 inputs N(0,1), seed 0).

    python -m turbogpt_b200.microbench                      # all kernels, one line each
    python -m turbogpt_b200.microbench --only gemm --iters 20
    python -m turbogpt_b200.microbench --only gemm --shape 32768,3072,768 --layout kk --iters 3

GEMM shapes are the step's projections at 32 768 tokens: (M,N,K) = (32768,3072,768),
(32768,768,3072), (32768,2304,768), (32768,768,768), their input-gradient forms (B read
MN-major) and weight-gradient forms (both operands MN-major, K = 32768).  Attention is causal,
B=32, H=12, T=1024, d_head=64 (FLOPs counted on the causal half).  Cross-entropy is 256-way over
[32768, 256] logits.  Times are CUDA-event averages after warm-up; every kernel's operands exceed
the 126 MB L2 or are rotated over several buffers so that they do.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import bridge


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e-3


def gemm_case(lib, m, n, k, layout, iters, out_fp32=False, tensor_cores=True):
    """layout: two letters, k = K-major, m = MN-major, for A then B."""
    g = torch.Generator(device="cuda").manual_seed(0)
    a_mn, b_mn = layout[0] == "m", layout[1] == "m"
    rotate = max(1, min(4, int(300e6 // ((m * k + n * k) * 2 + m * n * (4 if out_fp32 else 2))) + 1))
    a = [torch.randn((k, m) if a_mn else (m, k), generator=g, device="cuda").bfloat16() for _ in range(rotate)]
    b = [torch.randn((k, n) if b_mn else (n, k), generator=g, device="cuda").bfloat16() for _ in range(rotate)]
    c = [torch.empty(m, n, device="cuda", dtype=torch.float32 if out_fp32 else torch.bfloat16) for _ in range(rotate)]
    sa = (1, m) if a_mn else (k, 1)
    sb = (1, n) if b_mn else (k, 1)
    state = {"i": 0}

    def run():
        i = state["i"] = (state["i"] + 1) % rotate
        status = lib.tg_ex_gemm(a[i].data_ptr(), *sa, b[i].data_ptr(), *sb, c[i].data_ptr(), n, m, n, k,
                                int(out_fp32), int(tensor_cores), None)
        if status:
            raise RuntimeError(lib.tg_error().decode())

    seconds = _time(run, iters)
    return {"kernel": "gemm", "m": m, "n": n, "k": k, "layout": layout, "out": "fp32" if out_fp32 else "bf16",
            "us": seconds * 1e6, "tflops": 2.0 * m * n * k / seconds / 1e12}


def attention_case(lib, batch, context, heads, iters, backward, form=1):
    d_head, width = 64, heads * 64
    g = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn(batch * context, 3 * width, generator=g, device="cuda").bfloat16()
    dout = torch.randn(batch * context, width, generator=g, device="cuda").bfloat16()
    out = torch.empty(batch * context, width, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(batch * heads * context, device="cuda")
    dqkv = torch.empty_like(qkv)
    lib.tg_ex_attention_forward(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), batch, context, heads, d_head, 1, None)

    def forward():
        if lib.tg_ex_attention_forward(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), batch, context, heads, d_head,
                                       1, None):
            raise RuntimeError(lib.tg_error().decode())

    def back():
        if lib.tg_ex_attention_backward(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                        dqkv.data_ptr(), batch, context, heads, d_head, form, None):
            raise RuntimeError(lib.tg_error().decode())

    seconds = _time(back if backward else forward, iters)
    flops = 4.0 * batch * heads * context * context * d_head / 2 * (2.5 if backward else 1.0)
    name = ("attention_backward" if form == 1 else "attention_backward_single_pass") if backward else "attention_forward"
    return {"kernel": name, "batch": batch, "context": context,
            "heads": heads, "us": seconds * 1e6, "tflops": flops / seconds / 1e12}


def cross_entropy_case(lib, rows, iters):
    g = torch.Generator(device="cuda").manual_seed(0)
    rotate = 8  # 8 x 33.6 MB of logits + gradients: beyond L2
    logits = [torch.randn(rows, 256, generator=g, device="cuda").bfloat16() for _ in range(rotate)]
    grads = [torch.empty_like(l) for l in logits]
    targets = torch.randint(0, 256, (rows,), generator=g, device="cuda").to(torch.uint8)
    losses = torch.empty(rows, device="cuda")
    state = {"i": 0}

    def run():
        i = state["i"] = (state["i"] + 1) % rotate
        if lib.tg_ex_cross_entropy(logits[i].data_ptr(), targets.data_ptr(), losses.data_ptr(), grads[i].data_ptr(),
                                   rows, 1.0 / rows, None):
            raise RuntimeError(lib.tg_error().decode())

    seconds = _time(run, iters)
    bytes_moved = rows * 256 * 2 * 2 + rows * 5
    return {"kernel": "cross_entropy", "rows": rows, "us": seconds * 1e6, "gbs": bytes_moved / seconds / 1e9}


def split_fp32(values: torch.Tensor):
    """FP32 values as the engine stores them: high 16 bits (BF16) and low 16 bits, in separate arrays."""
    bits = values.contiguous().view(torch.int32)
    high = (bits >> 16).to(torch.int16).view(torch.bfloat16)
    low = (bits & 0xffff).to(torch.int16)
    return high.contiguous(), low.contiguous()


def norm_case(lib, rows, width, iters, backward):
    """LayerNorm forward (2 x rows x width x 2 B) or backward with the residual gradient
    (x, dy, residual in, dx out: 4 x rows x width x 2 B)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    rotate = 4  # 4 x 50 MB per tensor: beyond L2
    make = lambda: [torch.randn(rows, width, generator=g, device="cuda").bfloat16() for _ in range(rotate)]
    x, dy, res, out = make(), make(), make(), make()
    scale_high, scale_low = split_fp32(1 + .1 * torch.randn(width, generator=g, device="cuda"))
    bias_high, bias_low = split_fp32(.1 * torch.randn(width, generator=g, device="cuda"))
    dscale, dbias = torch.empty(width, device="cuda"), torch.empty(width, device="cuda")
    stats = [torch.empty(rows, 2, device="cuda") for _ in range(rotate)]
    state = {"i": 0}

    def forward():
        i = state["i"] = (state["i"] + 1) % rotate
        if lib.tg_ex_norm_forward(1, x[i].data_ptr(), scale_high.data_ptr(), scale_low.data_ptr(), bias_high.data_ptr(),
                                  bias_low.data_ptr(), out[i].data_ptr(), stats[i].data_ptr(), rows, width, None):
            raise RuntimeError(lib.tg_error().decode())

    def back():
        i = state["i"] = (state["i"] + 1) % rotate
        if lib.tg_ex_norm_backward(1, x[i].data_ptr(), dy[i].data_ptr(), scale_high.data_ptr(), scale_low.data_ptr(),
                                   res[i].data_ptr(), stats[i].data_ptr(), out[i].data_ptr(), dscale.data_ptr(),
                                   dbias.data_ptr(), rows, width, None):
            raise RuntimeError(lib.tg_error().decode())

    for _ in range(rotate):  # the backward pass reads the statistics the forward pass left
        forward()

    seconds = _time(back if backward else forward, iters)
    bytes_moved = rows * width * 2 * (4 if backward else 2)
    return {"kernel": "norm_backward" if backward else "norm_forward", "rows": rows, "width": width,
            "us": seconds * 1e6, "gbs": bytes_moved / seconds / 1e9}


def optimizer_case(iters):
    """The optimizer pass of BASELINE config 3 (85 M parameters: clip-norm reduction + one AdamW pass
    over gradient, momentum, variance and the two weight halves, 28 B + 4 B per parameter) through
    tg_optimizer_test, whose host copy of the gradient is outside the device-side profile."""
    base = bridge.Config(depth=12, context=64, batch=1, clip=1.0)
    ex = bridge.ConfigEx.gpt(base, 768, 12, flags=bridge.FLAG_PROFILE)
    with bridge.Native(ex) as engine:
        gradient = (np.random.default_rng(0).standard_normal(engine.count) * .01).astype(np.float32)
        engine.optimizer_test(gradient, 2)
        engine.profile(reset=True)
        engine.optimizer_test(gradient, iters)
        ms, launches = engine.profile()["optimizer"]
    seconds = ms * 1e-3 / iters
    return {"kernel": "sum_squares + adamw", "parameters": int(engine.count), "us": seconds * 1e6,
            "gbs": engine.count * 32 / seconds / 1e9}


def muon_case(iters):
    """Muon on the hidden matrices of BASELINE config 3's shapes (prepare, normalise, five Newton-Schulz
    iterations as batched tcgen05 GEMMs, apply) plus AdamW on the rest, through tg_optimizer_test."""
    base = bridge.Config(depth=12, context=64, batch=1, clip=1.0, ns_steps=5)
    ex = bridge.ConfigEx.gpt(base, 768, 12, flags=bridge.FLAG_PROFILE, hidden_optimizer=bridge.HIDDEN_MUON)
    with bridge.Native(ex) as engine:
        gradient = (np.random.default_rng(0).standard_normal(engine.count) * .01).astype(np.float32)
        engine.optimizer_test(gradient, 1)
        engine.profile(reset=True)
        engine.optimizer_test(gradient, iters)
        families = engine.profile()
    return {"kernel": "muon (5 Newton-Schulz iterations) + adamw", "parameters": int(engine.count),
            "muon_us": families["muon"][0] * 1e3 / iters, "muon_launches": families["muon"][1] // iters,
            "adamw_us": families["optimizer"][0] * 1e3 / iters}


def embedding_case(iters):
    """Embedding gather and its deterministic scatter-add inside a small engine (8 x 1024 tokens, d 768):
    a forward/backward pass through tg_batch, timed per kernel family."""
    base = bridge.Config(depth=1, context=1024, batch=8, clip=0)
    ex = bridge.ConfigEx.gpt(base, 768, 12, flags=bridge.FLAG_PROFILE)
    rng = np.random.default_rng(0)
    x = rng.integers(0, 256, (8, 1024), dtype=np.uint8)
    with bridge.Native(ex) as engine:
        engine.set_weights(bridge.initialize_weights(ex))
        engine.batch(x, x)
        engine.profile(reset=True)
        for _ in range(iters):
            engine.batch(x, x)
        families = engine.profile()
    tokens = 8 * 1024
    return {"kernel": "embedding gather / scatter", "tokens": tokens,
            "gather_us": families["embedding"][0] * 1e3 / iters, "scatter_us": families["embedding_backward"][0] * 1e3 / iters}


def predict_case(iters):
    """Latency of tg_predict on BASELINE config 3 (one 1024-byte context through 12 layers)."""
    import time
    base = bridge.Config(depth=12, context=1024, batch=32)
    context = np.random.default_rng(0).integers(0, 256, 1024, dtype=np.uint8)
    with bridge.Native(bridge.ConfigEx.gpt(base, 768, 12)) as engine:
        for _ in range(3):
            engine.predict(context)
        start = time.perf_counter()
        for _ in range(iters):
            engine.predict(context)
        seconds = (time.perf_counter() - start) / iters
    return {"kernel": "predict", "config": "12L-768d-ctx1024", "ms": seconds * 1e3,
            "note": "host call to host logits, one sequence"}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--only", default="all")
    parser.add_argument("--shape", default="")
    parser.add_argument("--layout", default="")
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--batch", type=int, default=32, help="sequences of the attention cases")
    parser.add_argument("--context", type=int, default=1024, help="tokens per sequence of the attention cases")
    args = parser.parse_args()
    lib = bridge.load_library()
    results = []
    tokens = 32768
    if args.only in ("all", "gemm"):
        if args.shape:
            m, n, k = (int(v) for v in args.shape.split(","))
            cases = [(m, n, k, args.layout or "kk")]
        else:
            cases = []
            for n, k in [(3072, 768), (768, 3072), (2304, 768), (768, 768)]:
                cases.append((tokens, n, k, "kk"))   # y = x W^T
                cases.append((tokens, k, n, "km"))   # dx = dy W
                cases.append((n, k, tokens, "mm"))   # dW = dy^T x
        for m, n, k, layout in cases:
            results.append(gemm_case(lib, m, n, k, layout, args.iters, out_fp32=layout == "mm"))
    if args.only in ("all", "attention", "attention_forward"):
        results.append(attention_case(lib, args.batch, args.context, 12, args.iters, False))
    if args.only in ("all", "attention", "attention_backward"):
        results.append(attention_case(lib, args.batch, args.context, 12, args.iters, True))
    if args.only in ("attention", "attention_backward_single_pass"):
        results.append(attention_case(lib, args.batch, args.context, 12, args.iters, True, form=2))
    if args.only in ("all", "cross_entropy"):
        results.append(cross_entropy_case(lib, tokens, args.iters))
    if args.only in ("all", "norm", "norm_forward"):
        results.append(norm_case(lib, tokens, 768, args.iters, False))
    if args.only in ("all", "norm", "norm_backward"):
        results.append(norm_case(lib, tokens, 768, args.iters, True))
    if args.only in ("all", "optimizer"):
        results.append(optimizer_case(min(args.iters, 8)))
    if args.only == "muon":
        results.append(muon_case(min(args.iters, 4)))
    if args.only == "embedding":
        results.append(embedding_case(min(args.iters, 8)))
    if args.only == "predict":
        results.append(predict_case(args.iters))
    for r in results:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
