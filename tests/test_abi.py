"""The C-ABI library loads without a GPU and exports every symbol include/lumen_b200.h declares; code
generation and NVRTC compilation (no device needed) work; compute entries fail loudly without a device."""

import ctypes
import os
import re

import pytest
import torch

from lumen_b200 import _lib, prims, tracer
from lumen_b200 import functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lumen_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    names = declared_symbols()
    assert "lb_fusion_launch" in names and "lb_last_error" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/lumen_b200.h but not exported"
    assert b"sm_100a" in lib.lb_version()


def test_fused_kernel_generates_and_compiles_without_a_gpu():
    def chain(x, g, b):
        y = F.relu(x * g + b)
        return y, prims.reduce_sum(y * y, (1,), "float32")

    g = tracer.trace(chain, ("bfloat16", (256, 4096)), ("bfloat16", (4096,)), ("bfloat16", (4096,)))
    handle = ctypes.c_void_p()
    _lib.check(_lib.lib().lb_fusion_compile(g.to_text().encode(), ctypes.byref(handle)))
    src = _lib.lib().lb_fusion_source(handle).decode()
    assert "fused_kernel" in src and "bf16x2_mul(" in src and "bf16x2_max(" in src and "__fadd_rn" in src
    assert _lib.lib().lb_fusion_num_inputs(handle) == 3 and _lib.lib().lb_fusion_num_outputs(handle) == 2


def test_only_a_summed_softmax_term_takes_the_short_exponential():
    """`exp(x - rowmax(x))` that is only summed (log-sum-exp) is generated as one multiply and one `ex2.approx`; the
    same exponential that also leaves the kernel (softmax) or one of anything else keeps `expf`."""

    def source(fn, *specs):
        handle = ctypes.c_void_p()
        _lib.check(_lib.lib().lb_fusion_compile(tracer.trace(fn, *specs).to_text().encode(), ctypes.byref(handle)))
        text = _lib.lib().lb_fusion_source(handle).decode()
        return text[text.index('extern "C" __global__'):]  # the kernel body, past the helper definitions

    def log_sum_exp(x):
        m = F.amax(x, -1, keepdim=True)
        return F.log(F.sum(F.exp(x - m), -1, keepdim=True)) + m

    spec = ("float32", (64, 512))
    lse = source(log_sum_exp, spec)
    assert "exp_sum_term(" in lse and "expf(" not in lse
    soft = source(lambda x: F.softmax(x, -1), spec)
    assert "expf(" in soft and "exp_sum_term(" not in soft
    plain = source(lambda x: F.sum(F.exp(x), -1), spec)
    assert "expf(" in plain and "exp_sum_term(" not in plain


def test_errors_are_statuses_with_messages():
    handle = ctypes.c_void_p()
    rc = _lib.lib().lb_fusion_compile(b"not a graph", ctypes.byref(handle))
    assert rc == 1 and b"cannot parse" in _lib.lib().lb_last_error()
    g = tracer.trace(lambda x: prims.reduce_sum(x, (1,), "float32"), ("float32", (4, 5, 6)))
    rc = _lib.lib().lb_fusion_compile(g.to_text().encode(), ctypes.byref(handle))
    assert rc == 2 and b"reduce_sum" in _lib.lib().lb_last_error()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_launch_without_a_gpu_fails_loudly():
    g = tracer.trace(lambda x: x + x, ("float32", (8,)))
    handle = ctypes.c_void_p()
    _lib.check(_lib.lib().lb_fusion_compile(g.to_text().encode(), ctypes.byref(handle)))
    buf = (ctypes.c_float * 8)()
    descs = (_lib.LbTensor * 2)(_lib.dense(ctypes.addressof(buf), "float32", (8,)), _lib.dense(ctypes.addressof(buf), "float32", (8,)))
    rc = _lib.lib().lb_fusion_launch(handle, descs, 2, None, None)
    assert rc == 3 and b"no CPU fallback" in _lib.lib().lb_last_error()
