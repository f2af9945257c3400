"""ctypes loader of the C-ABI library.  There is no fallback: if the library
is missing or a call fails, the caller gets a RuntimeError."""

from __future__ import annotations

import ctypes
import os
import threading

_LIB_PATH = os.environ.get("HALOPS_B200_LIB") or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), "lib", "libhalops_b200.so")
_lock = threading.Lock()
_tls = threading.local()
_lib = None

MODE_IDS = {"w8a8-mxfp8": 0, "w4a4-mxfp4": 1, "w4a4-nvfp4": 2}
GROUP_SIZE = {"w8a8-mxfp8": 32, "w4a4-mxfp4": 32, "w4a4-nvfp4": 16}

c_void_p, c_int, c_i64, c_size_t, c_char_p = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t, ctypes.c_char_p)

# name -> (restype, argtypes): exactly the entry points include/halops_b200.h declares
SIGNATURES = {
    "hq_parse_mode": (c_int, [c_char_p]),
    "hq_group_size": (c_int, [c_int]),
    "hq_sf_rows": (c_i64, [c_i64]),
    "hq_group_wise_quant": (c_int, [c_void_p, c_i64, c_int, c_i64, c_i64, c_int, c_int, c_int,
                                    c_void_p, c_void_p, c_int, c_void_p, c_char_p, c_size_t]),
    "hq_rms_norm_quant": (c_int, [c_void_p, c_i64, c_void_p, ctypes.c_float, c_i64, c_i64, c_int, c_int,
                                  c_void_p, c_void_p, c_int, c_void_p, c_char_p, c_size_t]),
    "hq_dense_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_char_p, c_size_t]),
    "hq_dense_gemm_situ_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, ctypes.c_float, ctypes.c_float,
                                         c_int, c_int, c_int, c_void_p, c_char_p, c_size_t]),
    "hq_batch_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_char_p, c_size_t]),
    "hq_group_masked_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_int,
                                     c_int, c_void_p, c_char_p, c_size_t]),
    "hq_group_contiguous_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                         c_int, c_int, c_void_p, c_char_p, c_size_t]),
    "hq_batch_gemm_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_i64,
                                    c_void_p, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int,
                                    c_int, c_int, c_void_p, c_char_p, c_size_t]),
    "hq_low_latency_gemm": (c_int, [c_void_p] * 10 + [c_i64] * 11 + [c_int, c_int, c_int, c_int, c_void_p, c_char_p,
                                                             c_size_t]),
    "hq_describe_group_tile": (c_int, [c_int, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_int, c_char_p,
                                       c_size_t]),
    "hq_sm_count": (c_int, [c_int]),
    "hq_device_status": (c_int, [c_int, c_void_p, ctypes.POINTER(ctypes.c_uint32), c_char_p, c_size_t]),
    "hq_selftest_bounded_wait": (c_int, [ctypes.c_uint32, c_int, c_void_p, c_char_p, c_size_t]),
    "hq_dense_gemm_allgather": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_int, c_int,
                                        c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_int, c_void_p,
                                        c_char_p, c_size_t]),
    "hq_dense_gemm_small_m_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_i64,
                                              c_i64, c_i64, c_i64, c_int, c_int, c_int, c_int, c_void_p, c_char_p,
                                              c_size_t]),
    "hq_selftest_decode_plan": (c_int, [c_i64, c_i64, c_int, c_int, c_char_p, c_size_t]),
    "hq_describe_tile": (c_int, [c_i64, c_i64, c_i64, c_int, c_int, c_int, c_char_p, c_size_t]),
    "hq_version": (c_char_p, []),
}


def lib_path() -> str:
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(_LIB_PATH):
                    raise RuntimeError(
                        f"halops_b200: native library not found at {_LIB_PATH}; build it with "
                        "`python -m halops_b200.build` (needs nvcc, no GPU). There is no CPU fallback.")
                handle = ctypes.CDLL(_LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def call(name: str, *args) -> None:
    """Calls an entry point whose last two parameters are (err, errlen) and
    raises RuntimeError with the library's message on a non-zero return."""
    err = getattr(_tls, "err", None)
    if err is None:
        err = _tls.err = ctypes.create_string_buffer(512)  # one per thread: entry points are re-entrant
    rc = getattr(lib(), name)(*args, err, 512)
    if rc != 0:
        raise RuntimeError(err.value.decode("utf-8", "replace") or f"{name} failed with code {rc}")


def current_stream(device) -> int:
    """Handle of torch's current CUDA stream on ``device`` (a ``torch.device`` with an index).
    ``torch.cuda.current_stream`` builds a Stream object for this, which costs the host several
    microseconds per call; torch's raw getter does not."""
    import torch

    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None and device.index is not None:
        return raw(device.index)
    return torch.cuda.current_stream(device).cuda_stream
