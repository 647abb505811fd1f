"""The C-ABI library loads without a GPU and exports every symbol that
include/jangq_b200.h declares; argument validation works without a device."""
import ctypes
import os
import re

import pytest

from jangq_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "jangq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jq_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from jangq_b200 import build
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_version_and_status_strings(lib):
    assert lib.jq_version() >= 100
    assert lib.jq_status_string(0) == b"ok"
    assert b"invalid" in lib.jq_status_string(_lib.JQ_EINVAL)


def test_argument_validation_needs_no_gpu(lib):
    # shape errors are detected on the host before anything touches the device
    rc = lib.jq_quantize(None, _lib.JQ_F16, 4, 100, 4, 64, _lib.JQ_F16, 0, None, None, None, None)
    assert rc == _lib.JQ_EINVAL and b"not divisible by group_size" in lib.jq_last_error()
    rc = lib.jq_quantize(None, _lib.JQ_F16, 4, 128, 7, 64, _lib.JQ_F16, 0, None, None, None, None)
    assert rc == _lib.JQ_EUNSUPPORTED
    rc = lib.jq_dequantize(None, None, None, _lib.JQ_F16, 4, 128, 4, 48, None, _lib.JQ_F32, None)
    assert rc == _lib.JQ_EUNSUPPORTED
    rc = lib.jq_qgemv(None, _lib.JQ_BF16, 99, 128, None, None, None, _lib.JQ_BF16, 16, 128, 4, 64, None,
                      _lib.JQ_BF16, 16, None)
    assert rc == _lib.JQ_EINVAL
    with pytest.raises(_lib.JangqError):
        _lib.check(rc)


def test_cpu_tensors_are_rejected():
    import torch
    import jangq_b200 as jq
    with pytest.raises(_lib.JangqError):
        jq.quantize(torch.zeros(4, 64), 64, 4)
