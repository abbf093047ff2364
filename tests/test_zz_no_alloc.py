"""`lb_attention_bwd_static`: the attention backward for callers that cannot allocate device memory at call time
(a fixed memory pool, a locked allocator, a latency budget). Its scratch is an array built into the library, so it
must give exactly what `lb_attention_bwd` gives with caller-provided scratch, call after call, and refuse problems
larger than that array. Collected last so that a run stopping at the first failure has run everything else."""

import ctypes

import numpy as np
import pytest
import torch

from lumen_b200 import _lib
from lumen_b200.runtime import attention_backward, attention_forward, current_stream, desc, device_status

pytestmark = pytest.mark.gpu


def backward_static(q, k, v, o, d_o, lse, causal):
    """Calls the allocation-free entry through the C ABI; the outputs are allocated here, by the test."""
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    d = _lib.LbAttnDesc()
    d.scale = float(q.shape[3] ** -0.5)
    d.causal = int(causal)
    d.causal_offset = k.shape[1] - q.shape[1]
    descs = [desc(t) for t in (q, k, v, o, d_o, lse, dq, dk, dv)]
    rc = _lib.lib().lb_attention_bwd_static(ctypes.byref(d), *[ctypes.byref(x) for x in descs], current_stream())
    return rc, (dq, dk, dv)


def operands(cuda, b, s, n, h, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn((b, s, n, h), generator=gen).bfloat16().to(cuda) for _ in range(4)]


def test_static_scratch_matches_caller_scratch_twice(cuda):
    """Two different problems in a row: the second call finds the first one's leftovers in the shared array and
    must not be affected by them. The kernels are the same and deterministic, so the results are bit-identical.
    `device_status()` reads the word the static entry's kernels raise as well as the library's own."""
    for seed, (b, s, n, h, causal) in enumerate([(2, 256, 2, 64, True), (1, 384, 3, 128, False)]):
        q, k, v, d_o = operands(cuda, b, s, n, h, seed)
        o, lse = attention_forward(q, k, v, causal=causal)
        want = attention_backward(q, k, v, o, d_o, lse, causal=causal)
        rc, got = backward_static(q, k, v, o, d_o, lse, causal)
        assert rc == 0, _lib.lib().lb_last_error()
        device_status()
        for a, w in zip(got, want):
            assert torch.isfinite(a.float()).all()
            np.testing.assert_array_equal(a.view(torch.uint16).cpu().numpy(), w.view(torch.uint16).cpu().numpy())


def test_static_entry_takes_no_device_memory_after_its_first_call(cuda):
    """The first call on a device loads the kernels and the built-in array (the driver materialises them then) and
    looks the array's address up; from the second call on the device's free memory does not move."""
    q, k, v, d_o = operands(cuda, 1, 256, 2, 64, 7)
    o, lse = attention_forward(q, k, v, causal=True)
    outs = [torch.empty_like(t) for t in (q, k, v)]
    d = _lib.LbAttnDesc()
    d.scale, d.causal, d.causal_offset = 0.125, 1, 0
    descs = [desc(t) for t in (q, k, v, o, d_o, lse, *outs)]
    args = [ctypes.byref(d), *[ctypes.byref(x) for x in descs], current_stream()]
    assert _lib.lib().lb_attention_bwd_static(*args) == 0, _lib.lib().lb_last_error()  # warm-up: one-time set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert _lib.lib().lb_attention_bwd_static(*args) == 0
    assert _lib.lib().lb_device_status() == 0  # synchronises; reads the static entry's status word, no allocation
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_a_timeout_in_the_static_entrys_word_is_reported(cuda):
    """The static entry's kernels raise a word of their own; `lb_device_status` must report and clear it. A one-CTA
    kernel that waits 100,000 cycles on a barrier nobody arrives on raises it (nothing faults or hangs)."""
    lib = _lib.lib()
    lib.lb_debug_wait_timeout.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    assert lib.lb_debug_wait_timeout(100_000, 1, current_stream()) == 0, lib.lb_last_error()
    assert lib.lb_device_status() == 4  # LB_ERR_TIMEOUT
    assert lib.lb_device_status() == 0  # cleared by the read


def test_static_scratch_rejects_what_does_not_fit(cuda):
    """batch * heads * query length beyond 1,048,576 rows is refused with a message naming the limit; nothing runs."""
    b, s, n, h = 1, 4096, 320, 64  # 1,310,720 rows; the tensors themselves are never touched
    q = torch.empty((b, s, n, h), dtype=torch.bfloat16, device=cuda)
    lse = torch.empty((b, n, s), dtype=torch.float32, device=cuda)
    rc, _ = backward_static(q, q, q, q, q, lse, True)
    assert rc == 1
    assert b"exceeds the built-in scratch" in _lib.lib().lb_last_error()
