"""Kernel-level GPU checks through the C-ABI microbenchmark entry points: the tcgen05 GEMM in
all operand layouts against an FP32 product, attention and cross-entropy against plain PyTorch."""
import numpy as np
import pytest
import torch

from turbogpt_b200 import load_library
from helpers import max_relative

pytestmark = pytest.mark.gpu
BACKWARD_ON_TENSOR_CORES = True


def gemm(lib, a, a_strides, b, b_strides, m, n, k, out_fp32, tensor_cores):
    c = torch.zeros(m, n, device="cuda", dtype=torch.float32 if out_fp32 else torch.bfloat16)
    status = lib.tg_ex_gemm(a.data_ptr(), *a_strides, b.data_ptr(), *b_strides, c.data_ptr(), n, m, n, k,
                            int(out_fp32), int(tensor_cores), None)
    assert status == 0, lib.tg_error().decode()
    torch.cuda.synchronize()
    return c.float().cpu().numpy()


def operands(m, n, k, a_mn, b_mn, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = torch.randn(n, k, generator=g).bfloat16()
    expected = (a.float() @ b.float().T).numpy()
    a_dev = (a.T.contiguous() if a_mn else a).cuda()   # MN-major: stored [k, m]
    b_dev = (b.T.contiguous() if b_mn else b).cuda()
    a_strides = (1, m) if a_mn else (k, 1)
    b_strides = (1, n) if b_mn else (k, 1)
    return a_dev, a_strides, b_dev, b_strides, expected


# forward (K-major, K-major), input gradient (K-major, MN-major), weight gradient (MN, MN)
LAYOUTS = [(False, False), (False, True), (True, True), (True, False)]


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (256, 256, 128), (384, 192, 320), (1000, 264, 200),
                                   (128, 768, 4096), (4096, 2304, 768),
                                   (200, 136, 8192)])  # ragged edges with many K splits (added by their own kernel)
def test_tensor_core_gemm_matches_fp32_product(a_mn, b_mn, m, n, k):
    lib = load_library()
    if a_mn and m % 8:
        pytest.skip("an MN-major A needs a multiple of 8 rows")
    a, sa, b, sb, expected = operands(m, n, k, a_mn, b_mn)
    for out_fp32 in (True, False):
        got = gemm(lib, a, sa, b, sb, m, n, k, out_fp32, True)
        # FP32 accumulation of exact BF16 products: only summation order differs.
        tolerance = 1e-5 if out_fp32 else 4e-3
        assert max_relative(got, expected) <= tolerance, (m, n, k, a_mn, b_mn, out_fp32)
        simt = gemm(lib, a, sa, b, sb, m, n, k, out_fp32, False)
        assert max_relative(simt, expected) <= tolerance


def test_split_k_weight_gradient_is_deterministic():
    lib = load_library()
    a, sa, b, sb, expected = operands(768, 768, 16384, True, True, seed=3)
    first = gemm(lib, a, sa, b, sb, 768, 768, 16384, True, True)
    assert max_relative(first, expected) <= 2e-5
    for _ in range(3):
        np.testing.assert_array_equal(first, gemm(lib, a, sa, b, sb, 768, 768, 16384, True, True))


def test_cross_entropy_matches_torch():
    lib = load_library()
    rows = 4096 + 3
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(rows, 256, generator=g).bfloat16()
    targets = torch.randint(0, 256, (rows,), generator=g).to(torch.uint8)
    expected_loss = torch.nn.functional.cross_entropy(logits.float(), targets.long(), reduction="none")
    probs = torch.softmax(logits.float(), -1)
    probs[torch.arange(rows), targets.long()] -= 1
    d_logits, d_targets = logits.cuda(), targets.cuda()
    losses = torch.empty(rows, device="cuda")
    grads = torch.empty(rows, 256, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / rows
    assert lib.tg_ex_cross_entropy(d_logits.data_ptr(), d_targets.data_ptr(), losses.data_ptr(), grads.data_ptr(),
                                   rows, scale, None) == 0
    torch.cuda.synchronize()
    np.testing.assert_allclose(losses.cpu().numpy(), expected_loss.numpy(), rtol=1e-5, atol=1e-5)
    assert max_relative(grads.float().cpu().numpy(), (probs * scale).numpy()) <= 4e-3


@pytest.mark.parametrize("rows,width", [(4096 + 3, 768), (300, 256), (33000, 768), (128, 64)])
def test_head_and_cross_entropy_in_one_kernel(rows, width):
    """The training step's head: logits stay in FP32 inside the kernel (cuda/model.cuh:31-58)."""
    lib = load_library()
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, width, generator=g, device="cuda").bfloat16()
    head = (torch.randn(256, width, generator=g, device="cuda") * (4.0 / width ** 0.5)).bfloat16()
    targets = torch.randint(0, 256, (rows,), generator=g, device="cuda").to(torch.uint8)
    losses = torch.empty(rows, device="cuda")
    grads = torch.empty(rows, 256, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / rows
    assert lib.tg_ex_head_cross_entropy(x.data_ptr(), head.data_ptr(), targets.data_ptr(), losses.data_ptr(),
                                        grads.data_ptr(), rows, width, scale, None) == 0, lib.tg_error()
    torch.cuda.synchronize()
    logits = x.double() @ head.double().T
    expected = torch.nn.functional.cross_entropy(logits, targets.long(), reduction="none")
    probabilities = torch.softmax(logits, -1)
    probabilities[torch.arange(rows), targets.long()] -= 1
    torch.testing.assert_close(losses.double(), expected, rtol=2e-5, atol=2e-5)
    assert max_relative(grads.float().cpu().numpy(), (probabilities * scale).float().cpu().numpy()) <= 4e-3
    # the loss alone (evaluation), and the same bits on a second call
    again = torch.empty_like(losses)
    assert lib.tg_ex_head_cross_entropy(x.data_ptr(), head.data_ptr(), targets.data_ptr(), again.data_ptr(), None,
                                        rows, width, scale, None) == 0, lib.tg_error()
    torch.cuda.synchronize()
    assert torch.equal(again, losses)


@pytest.mark.parametrize("batch,context,heads,d_head", [(2, 128, 2, 64), (1, 200, 3, 64), (2, 64, 2, 32),
                                                        (2, 1024, 2, 64), (3, 520, 1, 64), (1, 8, 1, 64),
                                                        (2, 40, 2, 64), (1, 65, 1, 64)])
def test_attention_matches_torch(batch, context, heads, d_head):
    lib = load_library()
    width = heads * d_head
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(batch * context, 3 * width, generator=g).bfloat16()
    dout = torch.randn(batch * context, width, generator=g).bfloat16()
    q, k, v = [t.reshape(batch, context, heads, d_head).transpose(1, 2).float().requires_grad_() for t in qkv.split(width, -1)]
    mask = torch.ones(context, context, dtype=torch.bool).tril()
    scores = (q @ k.transpose(-1, -2) / d_head ** .5).masked_fill(~mask, float("-inf"))
    out = torch.softmax(scores, -1) @ v
    out.backward(dout.reshape(batch, context, heads, d_head).transpose(1, 2).float())
    expected_out = out.detach().transpose(1, 2).reshape(batch * context, width).numpy()
    expected_dqkv = torch.cat([t.grad.transpose(1, 2).reshape(batch * context, width) for t in (q, k, v)], -1).numpy()
    d_qkv, d_dout = qkv.cuda(), dout.cuda()
    d_out = torch.empty(batch * context, width, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(batch * heads * context, device="cuda")
    d_dqkv = torch.empty_like(d_qkv)
    for tensor_cores in ((0, 1) if d_head == 64 else (0,)):
        d_out.zero_()
        lse.zero_()
        assert lib.tg_ex_attention_forward(d_qkv.data_ptr(), d_out.data_ptr(), lse.data_ptr(), batch, context, heads,
                                           d_head, tensor_cores, None) == 0, lib.tg_error()
        torch.cuda.synchronize()
        assert max_relative(d_out.float().cpu().numpy(), expected_out) <= 1e-2, tensor_cores
        expected_lse = torch.logsumexp(scores, -1).detach().reshape(-1).numpy()
        np.testing.assert_allclose(lse.cpu().numpy(), expected_lse, rtol=1e-4, atol=1e-4)
        if tensor_cores and not BACKWARD_ON_TENSOR_CORES:
            continue
        for form in ((1, 2) if tensor_cores else (0,)):  # 2: the single-pass tensor-core kernel
            d_dqkv.zero_()
            assert lib.tg_ex_attention_backward(d_qkv.data_ptr(), d_out.data_ptr(), d_dout.data_ptr(), lse.data_ptr(),
                                                d_dqkv.data_ptr(), batch, context, heads, d_head, form, None) == 0, \
                lib.tg_error()
            torch.cuda.synchronize()
            assert max_relative(d_dqkv.float().cpu().numpy(), expected_dqkv) <= 1e-2, form


@pytest.mark.parametrize("rows,width", [(1000, 768), (515, 256), (300, 1024), (64, 96)])
@pytest.mark.parametrize("kind", [0, 1])
def test_norms_match_torch(rows, width, kind):
    """RMSNorm / LayerNorm forward and backward (with the running residual gradient) as stand-alone
    kernels against FP32 PyTorch: outputs within one BF16 rounding, scale and bias gradients (FP32,
    fixed-order sums over rows) to 1e-4, and the same bits on a second call."""
    from turbogpt_b200.microbench import split_fp32
    lib = load_library()
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(rows, width, generator=g) * 2 + .3).bfloat16()
    dy = torch.randn(rows, width, generator=g).bfloat16()
    residual = torch.randn(rows, width, generator=g).bfloat16()
    scale = 1 + .2 * torch.randn(width, generator=g)
    bias = .1 * torch.randn(width, generator=g)
    xf = x.float().requires_grad_()
    sf, bf = scale.clone().requires_grad_(), bias.clone().requires_grad_()
    if kind == 1:
        expected = torch.nn.functional.layer_norm(xf, (width,), sf, bf, eps=1e-5)
    else:
        expected = torch.nn.functional.rms_norm(xf, (width,), sf, eps=1e-6)
    expected.backward(dy.float())
    d_x, d_dy, d_res = x.cuda(), dy.cuda(), residual.cuda()
    halves = [t.cuda() for t in (*split_fp32(scale), *split_fp32(bias))]
    y = torch.zeros_like(d_x)
    stats = torch.zeros(rows, 2, device="cuda")
    assert lib.tg_ex_norm_forward(kind, d_x.data_ptr(), halves[0].data_ptr(), halves[1].data_ptr(), halves[2].data_ptr(),
                                  halves[3].data_ptr(), y.data_ptr(), stats.data_ptr(), rows, width, None) == 0, lib.tg_error()
    torch.cuda.synchronize()
    assert max_relative(y.float().cpu().numpy(), expected.detach().numpy()) <= 2.0 ** -8
    results = []
    for saved in (stats.data_ptr(), stats.data_ptr(), None):  # twice with the saved statistics, once recomputing them
        dx = torch.zeros_like(d_x)
        dscale, dbias = torch.zeros(width, device="cuda"), torch.zeros(width, device="cuda")
        assert lib.tg_ex_norm_backward(kind, d_x.data_ptr(), d_dy.data_ptr(), halves[0].data_ptr(), halves[1].data_ptr(),
                                       d_res.data_ptr(), saved, dx.data_ptr(), dscale.data_ptr(), dbias.data_ptr(), rows,
                                       width, None) == 0, lib.tg_error()
        torch.cuda.synchronize()
        results.append((dx.float().cpu().numpy(), dscale.cpu().numpy(), dbias.cpu().numpy()))
    recomputed = results.pop()
    assert max_relative(recomputed[0], results[0][0]) <= 2.0 ** -7
    assert max_relative(recomputed[1], results[0][1]) <= 1e-4
    dx, dscale, dbias = results[0]
    expected_dx = residual.float() + xf.grad.bfloat16().float()  # rounded, then added to the residual gradient
    assert max_relative(dx, expected_dx.numpy()) <= 2.0 ** -7
    assert max_relative(dscale, sf.grad.numpy()) <= 1e-4
    if kind == 1:
        assert max_relative(dbias, bf.grad.numpy()) <= 1e-4
    for a, b in zip(*results):
        np.testing.assert_array_equal(a, b)
