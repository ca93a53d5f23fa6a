"""The allocation-free weight gradient (tg_ex_weight_gradient_static) against the ordinary GEMM
entry point.  It exists for hosts that cannot allocate device memory when the gradient is needed
(their own pool owns the GPU, or cudaMalloc's device-wide synchronisation is unaffordable there), so
its split-K scratch is an array built into the library.  Both entry points pick the same schedule
and run the same deterministic kernel, so the results must be bit-identical — on two calls in a row,
because the second call starts from the scratch contents the first one left behind — and the device's
free memory must not move across the second call.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from turbogpt_b200 import load_library

pytestmark = pytest.mark.gpu


def test_static_scratch_weight_gradient_matches_allocating_entry_point():
    lib = load_library()
    g = torch.Generator().manual_seed(7)
    for tokens, out, width in [(16384, 512, 512), (8192, 1024, 256), (4096, 768, 256)]:  # all take the split-K path
        dy = torch.randn(tokens, out, generator=g).bfloat16().cuda()
        x = torch.randn(tokens, width, generator=g).bfloat16().cuda()
        expected = torch.zeros(out, width, device="cuda")
        assert lib.tg_ex_gemm(dy.data_ptr(), 1, out, x.data_ptr(), 1, width, expected.data_ptr(), width,
                              out, width, tokens, 1, 1, None) == 0, lib.tg_error()
        torch.cuda.synchronize()
        reference = (dy.float().T @ x.float()).cpu().numpy()
        assert np.abs(expected.cpu().numpy() - reference).max() <= 2e-5 * np.abs(reference).max()
        outputs = [torch.full((out, width), float("nan"), device="cuda") for _ in range(2)]
        for call, got in enumerate(outputs):
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            assert lib.tg_ex_weight_gradient_static(dy.data_ptr(), x.data_ptr(), got.data_ptr(), out, width, tokens,
                                                    None) == 0, lib.tg_error()
            torch.cuda.synchronize()
            if call == 1:  # the first call on a device may create the CUDA module's lazily loaded state
                assert torch.cuda.mem_get_info()[0] == free_before
            np.testing.assert_array_equal(got.cpu().numpy(), expected.cpu().numpy(), err_msg=f"call {call}")
            np.testing.assert_allclose(got.cpu().numpy(), reference, atol=2e-5 * np.abs(reference).max())
        assert lib.tg_ex_last_device_error(None) == 0


def test_static_scratch_refuses_shapes_beyond_its_array():
    lib = load_library()
    tokens, out, width = 16384, 3072, 768  # 2 splits x 3072 x 768 floats = 18.9 MB > 16 MiB
    dy = torch.zeros(tokens, out, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(tokens, width, dtype=torch.bfloat16, device="cuda")
    dw = torch.zeros(out, width, device="cuda")
    status = lib.tg_ex_weight_gradient_static(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), out, width, tokens, None)
    message = lib.tg_error().decode()
    if status == 0:  # the tile search may pick an unsplit schedule, which needs no scratch
        pytest.skip("shape did not need scratch on this device")
    assert status < 0 and "built-in array holds" in message
