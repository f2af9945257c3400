"""``low_latency_mma_gemm``: same signature, defaults and error texts as the reference's
``halops.low_latency_mma_gemm`` (``halops/gemm/low_latency_mma_gemm.py:25-109``; host
checks of ``csrc/kernel/gemm/low_latency_utils.cuh:222-273`` and
``csrc/kernel/gemm/low_latency_mma_gemm.cu:23-76``), executed by this package's tcgen05
kernel for plain-layout scales through the C ABI."""

from __future__ import annotations

from typing import Optional

import torch

from .. import _native

__all__ = ["low_latency_mma_gemm"]


def _check(cond: bool, msg) -> None:
    """``msg``: the text, or a callable that builds it (only called when the check fails)."""
    if not cond:
        raise RuntimeError(msg() if callable(msg) else msg)


def _scale_ok(scale: torch.Tensor, rows: int) -> bool:
    return scale.dim() == 2 and scale.size(0) == rows and scale.stride(0) % 16 == 0 and scale.stride(1) == 1


def low_latency_mma_gemm(
    input: torch.Tensor,
    weight: torch.Tensor,
    sfa: torch.Tensor,
    sfb: torch.Tensor,
    output: torch.Tensor,
    input2: Optional[torch.Tensor] = None,
    weight2: Optional[torch.Tensor] = None,
    sfa2: Optional[torch.Tensor] = None,
    sfb2: Optional[torch.Tensor] = None,
    output2: Optional[torch.Tensor] = None,
    sm_count: int = -1,
    use_pdl: bool = True,
    use_sigmoid: bool = False,
) -> None:
    """W8A8-MXFP8 GEMM for decode-sized M (M <= 16): ``output = input @ weight^T``, with
    concat-K (``input2``: ``+ input2 @ weight2^T``) or dual output (``output2 = input @
    weight2^T``).

    Scales are the plain row-major ``[rows, K // 32]`` UE8M0 bytes of
    ``group_wise_quant(..., use_swizzle=False)`` with a row stride that is a multiple of 16
    bytes (a ``[rows, K // 32]`` view of a padded buffer otherwise).

    Args:
        input: [M, K1] float8_e4m3fn, M <= 16; K (K1 + K2) a multiple of 256.
        weight: [N, K1] float8_e4m3fn, N % 8 == 0.
        sfa / sfb: [M, K1 // 32] / [N, K1 // 32] uint8.
        output: [M, N] bfloat16, written in place.
        input2 / sfa2: [M, K2] and its scales, enables concat-K (K1 a multiple of 512).
        weight2 / sfb2: [N, K2] with ``input2``, [N2, K1] with ``output2`` (N2 % 8 == 0).
        output2: [M, N2] bfloat16, enables dual output; not combinable with ``input2``.
        sm_count: SMs to use (-1: all).
        use_pdl: launch with programmatic stream serialisation.
        use_sigmoid: write ``torch.sigmoid`` of the bfloat16 result instead; not with
            ``input2`` or ``output2``.
    """
    _check(
        (input2 is not None) == (sfa2 is not None) and (weight2 is not None) == (sfb2 is not None)
        and (weight2 is not None) == ((input2 is not None) != (output2 is not None)),
        "weight2 / sfb2 must come with either input2 / sfa2 or output2",
    )
    _check(input.dim() == 2 and weight.dim() == 2 and output.dim() == 2,
           "input, weight and output must be 2D tensors")
    m, n = input.size(0), weight.size(0)
    n2 = weight2.size(0) if output2 is not None else 0
    k1 = weight.size(1)
    k = k1 + (weight2.size(1) if input2 is not None else 0)
    _check(m <= 16, lambda: f"low_latency_mma_gemm supports M <= 16, got M={m}")
    _check(n % 8 == 0 and n2 % 8 == 0,
           lambda: f"low_latency_mma_gemm weight rows must be divisible by 8, got {n} and {n2}")
    _check(k % 256 == 0, lambda: f"low_latency_mma_gemm K must be divisible by 256, got K={k}")
    _check(input2 is None or input.size(1) % 512 == 0,
           lambda: f"concat-K K1 must be a multiple of 512, got K1={input.size(1)}")
    _check(
        _scale_ok(sfa, m) and _scale_ok(sfb, n) and (sfa2 is None or _scale_ok(sfa2, m))
        and (sfb2 is None or _scale_ok(sfb2, weight2.size(0))),
        lambda: "sfa / sfb / sfa2 / sfb2 must be plain row-major [rows, K / 32] scales "
        "(group_wise_quant(..., use_swizzle=False)) with a row stride that is a multiple of 16 bytes; got sfa "
        f"{list(sfa.shape)} strides {list(sfa.stride())}, sfb {list(sfb.shape)} strides {list(sfb.stride())}",
    )
    _check(not use_sigmoid or weight2 is None, "low_latency_mma_gemm use_sigmoid does not support input2 or output2")
    _check(input.size(1) == k1 and sfa.size(1) == k1 // 32 and sfb.size(1) == k1 // 32,
           lambda: f"input K must match weight K, got input K={input.size(1)}, weight K={k1}")
    _check(output.size(0) == m and output.size(1) == n and output.dtype == torch.bfloat16 and output.stride(1) == 1,
           lambda: f"output must be a bfloat16 [{m}, {n}] tensor with contiguous rows")
    tensors = [("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("output", output)]
    if input2 is not None:
        _check(input2.dim() == 2 and input2.size(0) == m and weight2.dim() == 2 and weight2.size(0) == n
               and input2.size(1) == weight2.size(1) and sfa2.size(1) == weight2.size(1) // 32
               and sfb2.size(1) == weight2.size(1) // 32,
               "input2 [M, K2], weight2 [N, K2] and their [rows, K2 / 32] scales must agree")
        tensors += [("input2", input2), ("sfa2", sfa2)]
    if output2 is not None:
        _check(weight2.dim() == 2 and weight2.size(1) == k1 and sfb2.size(1) == k1 // 32,
               "weight2 [N2, K1] and sfb2 [N2, K1 / 32] must match input's K")
        _check(output2.dim() == 2 and output2.size(0) == m and output2.size(1) == n2
               and output2.dtype == torch.bfloat16 and output2.stride(1) == 1,
               lambda: f"output2 must be a bfloat16 [{m}, {n2}] tensor with contiguous rows")
        tensors += [("output2", output2)]
    if weight2 is not None:
        tensors += [("weight2", weight2), ("sfb2", sfb2)]
    for name, t in tensors:
        _check(t.is_cuda, lambda: f"{name} must be a CUDA tensor (this library has no CPU path)")
    for name, t in tensors:
        if name in ("input", "weight", "input2", "weight2"):
            _check(t.is_contiguous(), lambda: f"{name} must be contiguous")

    def ptr(t):
        return None if t is None else t.data_ptr()

    _native.call(
        "hq_low_latency_gemm",
        input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), output.data_ptr(),
        ptr(input2), ptr(weight2), ptr(sfa2), ptr(sfb2), ptr(output2),
        m, n, n2, k1, k - k1, sfa.stride(0), sfb.stride(0),
        0 if sfa2 is None else sfa2.stride(0), 0 if sfb2 is None else sfb2.stride(0),
        output.stride(0) if m > 0 else max(n, 8), 0 if output2 is None else output2.stride(0),
        int(bool(use_sigmoid)), int(sm_count), int(bool(use_pdl)), input.device.index,
        _native.current_stream(input.device),
    )
