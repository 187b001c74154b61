"""The C-ABI library: loads, exports every symbol the header declares, and fails loudly
(never silently computes on the CPU) when there is no CUDA device."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT
from docc_b200 import _lib, build, ops

HEADER = os.path.join(ROOT, "include", "docc_b200", "rt.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(docc_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_and_current():
    assert os.path.exists(build.LIB_PATH), "run `python -m docc_b200.build`"
    assert build.is_current(), "libdocc_b200_rt.so is older than its sources"


def test_every_declared_symbol_is_exported_and_bound():
    handle = ctypes.CDLL(build.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 28
    for name in names:
        assert hasattr(handle, name), f"{name} declared in rt.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_strerror_table():
    handle = _lib.lib()
    assert handle.docc_b200_strerror(0) == b"ok"
    for code in range(1, 7):
        assert handle.docc_b200_strerror(code) not in (b"ok", b"unknown status")
    assert handle.docc_b200_strerror(99) == b"unknown status"


def test_no_torch_types_in_header():
    code = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)  # comments may mention torch layouts
    assert "torch" not in code and "at::" not in code and "#include <cuda" not in code


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_fails_loudly_without_a_device():
    handle = _lib.lib()
    assert handle.docc_b200_device_count() == 0
    assert handle.docc_b200_init(0) == 5  # DOCC_B200_ERR_NO_DEVICE
    x = np.random.rand(4, 4).astype(np.float32)
    with pytest.raises(_lib.DoccB200Error) as e:
        ops.softmax(x, [-1])
    assert e.value.status == 5
    with pytest.raises(_lib.DoccB200Error):
        ops.gemm(x, x)
    with pytest.raises(_lib.DoccB200Error):
        ops.conv(x.reshape(1, 1, 4, 4), x.reshape(1, 1, 4, 4))


def test_ops_reject_mixed_and_cpu_torch_inputs():
    x = np.zeros((2, 2), dtype=np.float32)
    with pytest.raises(TypeError):
        ops.gemm(x, torch.zeros(2, 2))
    with pytest.raises(TypeError):
        ops.softmax(torch.zeros(2, 2))  # CPU torch tensors are not silently accepted
    with pytest.raises(TypeError):
        ops.softmax(np.zeros((2, 2), dtype=np.int32))
