"""B200-native (sm_100a) block-scaled quantize -> dense GEMM path.

Drop-in for the reference's ``halops.group_wise_quant``, ``halops.dense_gemm``,
``halops.batch_gemm``, ``halops.group_masked_gemm``, ``halops.group_contiguous_gemm``,
``halops.low_latency_mma_gemm`` and ``halops.rms_norm_quant`` (plus ``interleave_gate_up`` and ``EpilogueOp``): same
Python signatures, executed by hand-written CUDA/PTX kernels through a C-ABI
shared library.  There is no CPU path and no fallback.
"""

from .gemm import (
    EpilogueOp,
    batch_gemm,
    dense_gemm,
    group_contiguous_gemm,
    group_masked_gemm,
    group_wise_quant,
    interleave_gate_up,
    low_latency_mma_gemm,
    rms_norm_quant,
)
from ._native import lib_path

__all__ = ["EpilogueOp", "batch_gemm", "dense_gemm", "group_contiguous_gemm", "group_masked_gemm",
           "group_wise_quant", "interleave_gate_up", "low_latency_mma_gemm", "rms_norm_quant", "device_status", "selftest_bounded_wait", "describe_tile",
           "describe_group_tile", "lib_path"]
__version__ = "0.1.0"


def device_status(device=None) -> int:
    """Synchronises the current stream of ``device`` and returns the device-side
    status word (0 = every bounded wait completed); raises RuntimeError when a
    kernel gave up on a wait."""
    import ctypes

    import torch

    from . import _native

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    status = ctypes.c_uint32(0)
    _native.call("hq_device_status", dev.index, torch.cuda.current_stream(dev).cuda_stream,
                 ctypes.byref(status))
    return int(status.value)


def selftest_bounded_wait(limit_us: int = 1000, device=None) -> None:
    """Launches the one-CTA kernel whose wait on a barrier nobody arrives on gives up after
    ``limit_us`` microseconds.  The next ``device_status`` raises (status 0x02), the one
    after it returns 0: the path a GEMM role takes when one of its waits times out."""
    import torch

    from . import _native

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _native.call("hq_selftest_bounded_wait", int(limit_us), dev.index, torch.cuda.current_stream(dev).cuda_stream)


def describe_tile(m: int, n: int, k: int, mode: str = "w8a8-mxfp8", sm_count: int = -1, device: int = -1) -> str:
    """The tile the GEMM dispatch picks for a shape (what the reference prints
    under ``IR_GEMM_TRACE``); raises the reference's "No dense ... tile" error
    for an illegal shape."""
    import ctypes

    from . import _native

    buf = ctypes.create_string_buffer(256)
    rc = _native.lib().hq_describe_tile(m, n, k, dict(_native.MODE_IDS, **{"w4a8-mxfp4": 3})[mode], sm_count, device, buf, len(buf))
    if rc != 0:
        raise RuntimeError(buf.value.decode())
    return buf.value.decode()


def describe_group_tile(kind: str, count: int, rows: int, n: int, k: int, mode: str = "w8a8-mxfp8",
                        total_m: int = -1, sm_count: int = -1, device: int = -1) -> str:
    """``describe_tile`` for ``batch_gemm`` / ``group_masked_gemm`` / ``group_contiguous_gemm``
    (``kind`` = "batch", "masked" or "contiguous"; ``rows`` per group, ``total_m`` rows in all,
    default ``count * rows``); raises the reference's "No <kind> ... tile" error for an
    illegal shape."""
    import ctypes

    from . import _native

    buf = ctypes.create_string_buffer(256)
    rc = _native.lib().hq_describe_group_tile(
        {"batch": 1, "masked": 2, "contiguous": 3}[kind], count, rows, count * rows if total_m < 0 else total_m,
        n, k, dict(_native.MODE_IDS, **{"w4a8-mxfp4": 3})[mode], sm_count, device, buf, len(buf))
    if rc != 0:
        raise RuntimeError(buf.value.decode())
    return buf.value.decode()
