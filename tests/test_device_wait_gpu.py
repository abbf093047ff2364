"""The wind-down path of the kernels' bounded waits, exercised without a fault: a wait that cannot complete runs out
of a SHORT budget, the kernel raises the device status word and returns normally, the host reads LB_ERR_TIMEOUT
once, and the context keeps working."""

import ctypes

import pytest
import torch

from lumen_b200 import _lib
from lumen_b200.runtime import current_stream, gemm

pytestmark = pytest.mark.gpu

LB_ERR_TIMEOUT = 4


def test_a_wait_that_runs_out_sets_the_status_word_and_the_context_survives(cuda):
    lib = _lib.lib()
    lib.lb_debug_wait_timeout.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    assert lib.lb_device_status() == 0
    assert lib.lb_debug_wait_timeout(100_000, 0, current_stream()) == 0, lib.lb_last_error()
    assert lib.lb_device_status() == LB_ERR_TIMEOUT
    assert b"wait ran out" in lib.lb_last_error()
    assert lib.lb_device_status() == 0  # read-and-clear
    # the context is intact: a tensor-core GEMM launched afterwards is right
    gen = torch.Generator(device="cpu").manual_seed(0)
    a = torch.randn((256, 320), generator=gen).bfloat16().to(cuda)
    b = torch.randn((320, 512), generator=gen).bfloat16().to(cuda)
    out = torch.empty((256, 512), dtype=torch.float32, device=cuda)
    gemm(a, b, out, kernel="tcgen05")
    want = a.float() @ b.float()
    assert lib.lb_device_status() == 0
    torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-3)


def test_the_budget_is_bounded(cuda):
    lib = _lib.lib()
    lib.lb_debug_wait_timeout.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    assert lib.lb_debug_wait_timeout(0, 0, None) == 1
    assert lib.lb_debug_wait_timeout(10**12, 0, None) == 1  # no long waits through this entry
    assert b"budget" in lib.lb_last_error()
