"""The C-ABI library loads without a GPU and exports every symbol include/b200i.h
declares; the Python host layer keeps the reference's refusals; the product
path fails loudly when no device is visible (no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

from mojolearn_b200 import _native, linalg, lowbit

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200i.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200i_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = _declared()
    assert len(names) >= 20
    lib = ctypes.CDLL(_native.LIB_PATH)
    for name in names:
        assert hasattr(lib, name), name


def test_python_binding_covers_the_header():
    declared = set(_declared())
    bound = set(_native.SIGNATURES) | set(_native.STRING_FUNCTIONS) | set(_native.POINTER_FUNCTIONS)
    assert declared == bound


def test_identity_of_the_binary():
    l = _native.lib()
    assert l.b200i_abi() == 1 and l.b200i_numeric_mode() == 1 and l.b200i_profile_version() == 1
    assert l.b200i_numerical_profile() == b"mojolearn.identical.gemm.fp32.v1" and l.b200i_vendor() == b"cuda"
    p = linalg.profile()
    assert p["profile"] == linalg.PROFILE and p["identity_claimed"] and linalg.numeric_mode() == "identical"
    linalg.require_identical()


def test_refusals_of_the_python_surface():
    f = np.zeros((4, 4), np.float32)
    with pytest.raises(TypeError):
        linalg.matmul(f.astype(np.float64), f)
    with pytest.raises(ValueError):
        linalg.matmul(f, f, transpose_a=True, transpose_b=True)
    with pytest.raises(ValueError):
        linalg.matmul(np.zeros((4, 3), np.float32), f)
    with pytest.raises(ValueError):
        linalg.matmul(f, f, out=np.zeros((3, 4), np.float32))
    with pytest.raises(TypeError):
        linalg.matmul(f, f, out=np.zeros((4, 4), np.float64))
    with pytest.raises(ValueError):
        linalg.matmul(np.zeros((0, 4), np.float32), f)
    with pytest.raises(ValueError):
        linalg.matmul_int8((np.zeros((2, 131073), np.int8), np.zeros(2, np.int32)),
                           (np.zeros((2, 131073), np.int8), np.zeros(2, np.int32)))
    with pytest.raises(ValueError):
        lowbit.pack_one(f[:, 0], "bfloat16")
    with pytest.raises(ValueError):
        lowbit.pack_one(f, "float16")
    with pytest.raises(ValueError):
        lowbit.format_of({"a": lowbit.BF16Weight(np.zeros((2, 2), np.uint16)),
                          "b": lowbit.Int8Weight(np.zeros((2, 2), np.int8), np.zeros(2, np.int32))})
    assert lowbit.format_of({"w": f}) == "float32" and not lowbit.is_packed(f)


def test_c_abi_refusals_need_no_gpu_for_bad_arguments():
    """Argument checks that come before any CUDA call: a negative count."""
    buf = ctypes.create_string_buffer(256)
    l = _native.lib()
    assert l.b200i_to_bf16(-1, None, None, None, -5, ctypes.cast(buf, ctypes.c_void_p), 256) == 1
    assert b"negative" in buf.value
    assert l.b200i_workspace_bytes(0, 4, 4) == 0


def test_no_cpu_fallback_without_a_device():
    if _native.lib().b200i_device_count() > 0:
        pytest.skip("a CUDA device is visible")
    f = np.zeros((4, 4), np.float32)
    with pytest.raises(_native.NativeError):
        linalg.matmul(f, f)
    with pytest.raises(_native.NativeError):
        linalg.to_bf16(f)
