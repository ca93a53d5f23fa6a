"""Parity at the sizes BASELINE names for the kernel microbenchmarks (single B200, BF16 inputs
N(0,1) from seed 0, FP32 accumulation): the three projection GEMMs at 32 768 tokens with their
input-gradient and weight-gradient forms against an FP32 product, causal attention forward and
backward at batch 32 x 12 heads x 1024 positions x 64 against the FP32 formula on sampled heads
(and one 4096-position case), cross-entropy over [32768, 256], and device sampling at contexts 256
and 1024 for rank 1 of 2.  All through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import indexing
from turbogpt_b200 import Config, ConfigEx, Native, bridge, load_library

pytestmark = pytest.mark.gpu
TOKENS = 32768


def _max_relative(a, b):
    return float((a - b).abs().max() / b.abs().max())


def _gemm(lib, a, sa, b, sb, m, n, k, out_fp32):
    c = torch.empty(m, n, device="cuda", dtype=torch.float32 if out_fp32 else torch.bfloat16)
    assert lib.tg_ex_gemm(a.data_ptr(), *sa, b.data_ptr(), *sb, c.data_ptr(), n, m, n, k, int(out_fp32), 1,
                          None) == 0, lib.tg_error().decode()
    torch.cuda.synchronize()
    return c


@pytest.mark.parametrize("out_features,in_features", [(3072, 768), (768, 3072), (2304, 768)])
def test_projection_gemms_at_32768_tokens(out_features, in_features):
    """y = x W^T (K-major, K-major), dx = dy W (B read MN-major), dW = dy^T x (both MN-major, FP32 out,
    split K) for one layer shape: the whole result against torch's FP32 product on the device (TF32
    off), and 48 sampled rows against a float64 product on the host."""
    torch.backends.cuda.matmul.allow_tf32 = False
    lib = load_library()
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(TOKENS, in_features, generator=g, device="cuda").bfloat16()
    w = torch.randn(out_features, in_features, generator=g, device="cuda").bfloat16()
    dy = torch.randn(TOKENS, out_features, generator=g, device="cuda").bfloat16()
    rows = torch.randperm(TOKENS, generator=torch.Generator().manual_seed(1))[:48]

    y = _gemm(lib, x, (in_features, 1), w, (in_features, 1), TOKENS, out_features, in_features, False)
    assert _max_relative(y.float(), x.float() @ w.float().T) <= 4e-3
    exact = x[rows.cuda()].double().cpu() @ w.double().cpu().T
    assert _max_relative(y[rows.cuda()].double().cpu(), exact) <= 4e-3

    dx = _gemm(lib, dy, (out_features, 1), w, (1, in_features), TOKENS, in_features, out_features, False)
    assert _max_relative(dx.float(), dy.float() @ w.float()) <= 4e-3
    exact = dy[rows.cuda()].double().cpu() @ w.double().cpu()
    assert _max_relative(dx[rows.cuda()].double().cpu(), exact) <= 4e-3

    dw = _gemm(lib, dy, (1, out_features), x, (1, in_features), out_features, in_features, TOKENS, True)
    # two FP32 sums of 32 768 products in different orders: each is ~1e-5 from the exact value
    assert _max_relative(dw, dy.float().T @ x.float()) <= 1e-4
    picked = rows[:48] % out_features
    exact = dy[:, picked.cuda()].double().cpu().T @ x.double().cpu()
    assert _max_relative(dw[picked.cuda()].double().cpu(), exact) <= 3e-5
    again = _gemm(lib, dy, (1, out_features), x, (1, in_features), out_features, in_features, TOKENS, True)
    assert torch.equal(dw, again)  # split K sums in a fixed order


def _attention_reference(qkv, dout, batch, context, heads, pairs):
    """FP32 causal attention forward and backward for the sampled (batch, head) pairs."""
    width = heads * 64
    q, k, v = [t.reshape(batch, context, heads, 64) for t in qkv.split(width, -1)]
    d = dout.reshape(batch, context, heads, 64)
    mask = torch.ones(context, context, dtype=torch.bool, device=qkv.device).tril()
    expected = {}
    for b, h in pairs:
        qq, kk, vv = [t[b, :, h].float().clone().requires_grad_() for t in (q, k, v)]
        scores = (qq @ kk.T / 8.0).masked_fill(~mask, float("-inf"))
        out = torch.softmax(scores, -1) @ vv
        out.backward(d[b, :, h].float())
        expected[(b, h)] = (out.detach(), torch.logsumexp(scores, -1).detach(), qq.grad, kk.grad, vv.grad)
    return expected


@pytest.mark.parametrize("form", [1, 2], ids=["engine_form", "single_pass"])
@pytest.mark.parametrize("batch,context,heads", [(32, 1024, 12), (2, 4096, 2)])
def test_attention_at_benchmark_size(batch, context, heads, form):
    lib = load_library()
    width = heads * 64
    g = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn(batch * context, 3 * width, generator=g, device="cuda").bfloat16()
    dout = torch.randn(batch * context, width, generator=g, device="cuda").bfloat16()
    out = torch.zeros(batch * context, width, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(batch * heads * context, device="cuda")
    dqkv = torch.zeros_like(qkv)
    assert lib.tg_ex_attention_forward(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), batch, context, heads, 64, 1,
                                       None) == 0, lib.tg_error()
    assert lib.tg_ex_attention_backward(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                        dqkv.data_ptr(), batch, context, heads, 64, form, None) == 0, lib.tg_error()
    torch.cuda.synchronize()
    pairs = sorted({(0, 0), (batch - 1, heads - 1), (batch // 2, heads // 2), (1, heads - 1), (batch - 1, 0)})
    expected = _attention_reference(qkv, dout, batch, context, heads, pairs)
    o = out.reshape(batch, context, heads, 64)
    dq, dk, dv = [t.reshape(batch, context, heads, 64) for t in dqkv.split(width, -1)]
    stats = lse.reshape(batch, heads, context)
    for (b, h), (e_out, e_lse, e_dq, e_dk, e_dv) in expected.items():
        assert _max_relative(o[b, :, h].float(), e_out) <= 1e-2, (b, h)
        torch.testing.assert_close(stats[b, h], e_lse, rtol=1e-4, atol=1e-4)
        assert _max_relative(dq[b, :, h].float(), e_dq) <= 1e-2, (b, h)
        assert _max_relative(dk[b, :, h].float(), e_dk) <= 1e-2, (b, h)
        assert _max_relative(dv[b, :, h].float(), e_dv) <= 1e-2, (b, h)
    assert torch.isfinite(out.float()).all() and torch.isfinite(dqkv.float()).all()
    # deterministic: a second backward gives the same bits
    again = torch.zeros_like(qkv)
    assert lib.tg_ex_attention_backward(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                        again.data_ptr(), batch, context, heads, 64, form, None) == 0, lib.tg_error()
    torch.cuda.synchronize()
    assert torch.equal(again, dqkv)


def test_cross_entropy_at_32768_rows():
    lib = load_library()
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.randn(TOKENS, 256, generator=g, device="cuda").bfloat16()
    targets = torch.randint(0, 256, (TOKENS,), generator=g, device="cuda").to(torch.uint8)
    losses = torch.empty(TOKENS, device="cuda")
    grads = torch.empty_like(logits)
    scale = 1.0 / TOKENS
    assert lib.tg_ex_cross_entropy(logits.data_ptr(), targets.data_ptr(), losses.data_ptr(), grads.data_ptr(),
                                   TOKENS, scale, None) == 0, lib.tg_error()
    torch.cuda.synchronize()
    expected = torch.nn.functional.cross_entropy(logits.float(), targets.long(), reduction="none")
    probabilities = torch.softmax(logits.float(), -1)
    probabilities[torch.arange(TOKENS), targets.long()] -= 1
    torch.testing.assert_close(losses, expected, rtol=1e-5, atol=1e-5)
    assert _max_relative(grads.float(), probabilities * scale) <= 4e-3


@pytest.mark.parametrize("context,batch", [(256, 8), (1024, 32)])
def test_sampling_at_long_contexts_for_rank_1_of_2(context, batch):
    """cuda/dataset.cuh:9-29 with lo = max(8, context), applied to the global batch: rank 1 of 2
    draws global sequences batch .. 2*batch-1, bit for bit what the C restatement draws."""
    data = np.random.default_rng(718).integers(0, 256, 1 << 20, dtype=np.uint8)
    base = Config(depth=1, context=context, batch=batch, seed=3407)
    ex = ConfigEx.gpt(base, 64, 1, world=2, rank=1, flags=bridge.FLAG_NO_COMMUNICATOR)
    with Native(ex) as engine:
        engine.set_data(data)
        for step in (0, 1, 7, 123456):
            x, y = engine.sample(step)
            ex_x, ex_y = indexing.byte_batch_c(data, 3407, step, batch, context, world=2, rank=1)
            np.testing.assert_array_equal(x, ex_x)
            np.testing.assert_array_equal(y, ex_y)
            whole = indexing.byte_batch_c(data, 3407, step, 2 * batch, context)[0]
            np.testing.assert_array_equal(x, whole[batch:])
        assert engine.lib.tg_train(engine.handle, 1) < 0 and b"communicator" in engine.lib.tg_error()
