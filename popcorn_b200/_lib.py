"""ctypes binding of libpopcorn_b200.so (the C ABI declared in include/popcorn_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be
bound, importing an op raises.  The reference reaches its own CUDA kernel
through a pybind11 module JIT-built on first use (src/popcorn/impls/_cuda.py:17-23,
src/popcorn/impls/swiglu_cu.py:8-23); here the library is prebuilt in-tree by
`python -m popcorn_b200.build`.
"""

from __future__ import annotations

import ctypes
import functools
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libpopcorn_b200.so"
ABI_VERSION = 1

F32, F16, BF16 = 0, 1, 2

_i64 = ctypes.c_int64
_int = ctypes.c_int
_ptr = ctypes.c_void_p
_dbl = ctypes.c_double
_size = ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/popcorn_b200.h declaration by declaration
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "b200_version": (_int, []),
    "b200_status_string": (ctypes.c_char_p, [_int]),
    "b200_last_error": (ctypes.c_char_p, []),
    "b200_launch_count": (ctypes.c_uint64, []),
    "b200_wait_timeouts": (ctypes.c_uint64, []),
    "b200_rms_norm": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _dbl, _ptr]),
    "b200_add_rms_norm": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _dbl, _ptr]),
    "b200_rms_norm_backward_scratch_bytes": (_int, [_i64, _i64, _int, ctypes.POINTER(_size)]),
    "b200_rms_norm_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _ptr, _size, _ptr]),
    "b200_add_rms_norm_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _dbl, _ptr, _size, _ptr]),
    "b200_rope": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _ptr]),
    "b200_rope_qk": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _ptr]),
    "b200_rope_paired": (_int, [_ptr] * 6 + [_i64] * 18 + [_int, _ptr]),
    "b200_qk_norm_rope": (_int, [_ptr] * 8 + [_i64] * 18 + [_dbl, _int, _ptr]),
    "b200_llama4_rope": (_int, [_ptr] * 5 + [_i64] * 17 + [_int, _ptr]),
    "b200_qk_norm_rope_backward_scratch_bytes": (_int, [_i64, _i64, _i64, _int, ctypes.POINTER(_size)]),
    "b200_qk_norm_rope_backward": (_int, [_ptr] * 12 + [_i64] * 12 + [_dbl, _int, _ptr, _size, _ptr]),
    "b200_swiglu": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_geglu": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_rms_norm_gated": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _int, _dbl, _ptr]),
    "b200_l2_norm": (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _int, _dbl, _ptr]),
    "b200_layer_norm": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _dbl, _ptr]),
    "b200_l2_norm_backward": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _ptr]),
    "b200_layer_norm_backward_scratch_bytes": (_int, [_i64, _i64, ctypes.POINTER(_size)]),
    "b200_layer_norm_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _ptr, _size, _ptr]),
    "b200_swiglu_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_geglu_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_sigmoid_gate_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_route": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_index_scratch_bytes": (_int, [_i64, _i64, _i64, ctypes.POINTER(_size)]),
    "b200_moe_index": (_int, [_ptr, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "b200_moe_route_index": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _ptr, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "b200_moe_index_static": (_int, [_ptr, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "b200_moe_index_static_max_bytes": (_int, [ctypes.POINTER(_size)]),
    "b200_moe_permute": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_gather": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_unpermute": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_unpermute_backward": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_grouped_gemm": (_int, [_ptr] * 5 + [_i64] * 6 + [_int, _ptr]),
    "b200_moe_grouped_gemm_gathered": (_int, [_ptr] * 6 + [_i64] * 7 + [_int, _ptr]),
    "b200_moe_grouped_gemm_gate_up": (_int, [_ptr] * 5 + [_i64] * 6 + [_int, _ptr]),
    "b200_moe_grouped_gemm_dgrad": (_int, [_ptr] * 6 + [_i64] * 6 + [_int, _ptr]),
    "b200_moe_grouped_gemm_wgrad": (_int, [_ptr] * 4 + [_i64] * 6 + [_int, _ptr]),
    "b200_moe_ep_destinations": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _ptr, _ptr]),
    "b200_moe_ep_meta_bytes": (_int, [ctypes.POINTER(_size)]),
    "b200_moe_ep_exchange": (_int, [_ptr, ctypes.POINTER(_ptr), _i64, _i64, _i64, _i64, ctypes.c_int32, _i64, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "b200_moe_ep_barrier": (_int, [ctypes.POINTER(_ptr), _i64, _i64, _i64, ctypes.c_int32, _i64, _ptr, _ptr]),
    "b200_moe_permute_multi": (_int, [_ptr, _ptr, _ptr, ctypes.POINTER(_ptr), _i64, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
    "b200_moe_unpermute_multi": (_int, [ctypes.POINTER(_ptr), _i64, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _int, _ptr]),
}


class B200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, function: str, status: int, name: str, detail: str) -> None:
        super().__init__(f"{function} failed with {name} ({status}): {detail}")
        self.function = function
        self.status = status
        self.status_name = name
        self.detail = detail


@functools.cache
def library() -> ctypes.CDLL:
    """Load the shared library once and bind every declared symbol."""
    if not LIBRARY_PATH.exists():
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build it with `python -m popcorn_b200.build` "
            "(needs nvcc; there is no non-CUDA implementation of these ops)"
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as error:
            raise ImportError(f"{LIBRARY_PATH} does not export {name}; rebuild it") from error
        fn.restype = restype
        fn.argtypes = argtypes
    found = lib.b200_version()
    if found != ABI_VERSION:
        raise ImportError(f"{LIBRARY_PATH} has ABI version {found}, this package expects {ABI_VERSION}; rebuild it")
    return lib


def call(name: str, *args: object) -> None:
    """Invoke a status-returning entry point and raise B200Error on failure."""
    lib = library()
    status = getattr(lib, name)(*args)
    if status != 0:
        raise B200Error(name, status, lib.b200_status_string(status).decode(), lib.b200_last_error().decode())


def launch_count() -> int:
    return int(library().b200_launch_count())


def wait_timeouts() -> int:
    """Bounded waits that ran out on the current device (0 unless a copy never landed); synchronises."""
    return int(library().b200_wait_timeouts())
