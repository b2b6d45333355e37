"""The C ABI without a GPU: the library loads, exports what the header declares, its host
arithmetic matches the oracle bit for bit, and it refuses loudly when there is no device."""
import ctypes
import os
import re

import numpy as np
import pytest

from loadngo_b200 import compute
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "cuda_compute.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cc_[a-z0-9_]+)\s*\(", text)) - {"cc_completion_fn"})


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(compute.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 35
    for name in names:
        assert hasattr(L, name), f"{name} is declared in cuda_compute.h but not exported"
    # and the ctypes mirror types exactly that set
    assert sorted(compute.SYMBOLS) == names


def test_host_rope_table_is_bit_identical_to_the_oracle():
    for kwargs, orc in [
        (dict(), oracle.Rope()),
        (dict(head_dim=32, original_context=64.0), oracle.Rope(32, 150000.0, 32.0, 64.0)),
        (dict(factor=1.0), oracle.Rope(64, 150000.0, 1.0, 4096.0)),
    ]:
        inv, scale = compute.yarn_inv_freq(**kwargs)
        want_inv, want_scale = orc.inv_freq()
        assert np.array_equal(inv, want_inv) and scale == want_scale
        for start, rows in [(0, 5), (4090, 12), (131000, 3)]:
            assert np.array_equal(compute.rope_table(start, rows, **kwargs), orc.table(start, rows))


def test_rope_rejects_bad_parameters():
    with pytest.raises(compute.DispatchError):
        compute.rope_table(0, 1, head_dim=63)
    with pytest.raises(compute.DispatchError):
        compute.rope_table(0, 1, theta=0.5)


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(compute.NoDevice):
        compute.Gpu(0)
    # raw entries validate before touching the device
    args = compute.DecodeArgs()
    with pytest.raises(compute.DispatchError):
        compute.check(compute.lib().cc_attention_decode_paged(None, ctypes.byref(args)))


def test_status_codes_mirror_the_reference_error_enum():
    # metal-compute/src/lib.rs:42-53
    assert [c.code for c in (compute.NoDevice, compute.Compile, compute.Alloc, compute.DispatchError,
                             compute.GpuError)] == [1, 2, 3, 4, 5]
