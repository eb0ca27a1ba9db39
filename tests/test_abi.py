"""The C-ABI library loads and exports what include/popcorn_b200.h declares.

No kernel is launched here: only argument validation, which returns before the
device is touched, and the loud failure on a machine without a usable GPU.
"""

import ctypes
import re
from pathlib import Path

import pytest
import torch

from popcorn_b200 import _lib

HEADER = Path(__file__).resolve().parents[1] / "include" / "popcorn_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_functions() == sorted(_lib.SIGNATURES)


def test_every_declared_symbol_is_exported(built_library):
    lib = ctypes.CDLL(str(built_library))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_version_and_status_strings(built_library):
    lib = _lib.library()
    assert lib.b200_version() == _lib.ABI_VERSION
    names = {lib.b200_status_string(code).decode() for code in range(8)}
    assert len(names) == 8 and "B200_OK" in names
    assert lib.b200_status_string(99).decode() == "B200_ERR_UNKNOWN"


def test_argument_validation_needs_no_device(built_library):
    null = ctypes.c_void_p(0)
    fake = ctypes.c_void_p(4096)  # never dereferenced: validation fails first
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_rms_norm", fake, fake, null, fake, -1, 8, 8, 8, _lib.F32, 1e-6, null)
    assert err.value.status_name == "B200_ERR_SHAPE"
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_rms_norm", null, fake, null, fake, 4, 8, 8, 8, _lib.F32, 1e-6, null)
    assert err.value.status_name == "B200_ERR_NULL_POINTER" and "x is NULL" in err.value.detail
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_swiglu", fake, fake, fake, 4, 8, 8, 8, 8, 7, null)
    assert err.value.status_name == "B200_ERR_DTYPE"
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_swiglu", fake, fake, fake, 4, 8, 4, 8, 8, _lib.BF16, null)
    assert err.value.status_name == "B200_ERR_SHAPE"
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_swiglu", ctypes.c_void_p(4097), fake, fake, 4, 8, 8, 8, 8, _lib.BF16, null)
    assert err.value.status_name == "B200_ERR_ALIGNMENT"
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_moe_route", fake, fake, fake, 4, 2048, 2, 2048, _lib.F32, null)
    assert err.value.status_name == "B200_ERR_SHAPE"
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_rope", fake, fake, fake, fake, 1, 4, 2, 16, 9, 128, 32, 16, 128, 32, 16, _lib.BF16, _lib.F32, 0, null)
    assert err.value.status_name == "B200_ERR_SHAPE"
    # zero-sized problems are accepted without touching anything
    _lib.call("b200_swiglu", null, null, null, 0, 8, 8, 8, 8, _lib.BF16, null)
    _lib.call("b200_moe_permute", null, null, null, 0, 2, 64, 64, 64, _lib.BF16, null)


def test_scratch_size_query(built_library):
    need = ctypes.c_size_t(0)
    _lib.call("b200_moe_index_scratch_bytes", 65536, 8, 64, ctypes.byref(need))
    header = 8 * (256 + 64)  # generation word, per-CTA flags and go word of the one-launch kernel
    assert need.value == header + (65536 * 8 // 2048) * 64 * 4
    _lib.call("b200_moe_index_scratch_bytes", 4096, 1, 64, ctypes.byref(need))   # 2 blocks of pairs, 64 CTAs of tokens
    assert need.value == header + 64 * 64 * 4
    _lib.call("b200_moe_index_scratch_bytes", 4096, 1, 1024, ctypes.byref(need))  # beyond the one-launch kernel: blocks only
    assert need.value == header + 2 * 1024 * 4
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_moe_index", ctypes.c_void_p(4096), 16, 2, 8, ctypes.c_void_p(4096), ctypes.c_void_p(4096),
                  ctypes.c_void_p(4096), ctypes.c_void_p(4096), ctypes.c_void_p(4096), ctypes.c_size_t(4), ctypes.c_void_p(0))
    assert err.value.status_name == "B200_ERR_SCRATCH"


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the failure mode of a machine without a GPU")
def test_compute_call_without_gpu_fails_loudly(built_library):
    fake = ctypes.c_void_p(4096)
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_swiglu", fake, fake, fake, 4, 8, 8, 8, 8, _lib.BF16, ctypes.c_void_p(0))
    assert err.value.status_name == "B200_ERR_DEVICE"
