"""``rms_norm_quant``: same signature, shapes and error texts as the reference's
``halops.rms_norm_quant`` (``halops/gemm/rms_norm_quant.py:26-65``; host checks of
``csrc/kernel/gemm/rms_norm_quant.cu:111-155``), executed by this package's
sm_100a kernel through the C ABI."""

from __future__ import annotations

from typing import Tuple

import torch

from .. import _native

__all__ = ["rms_norm_quant"]


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def rms_norm_quant(
    input: torch.Tensor,
    weight: torch.Tensor,
    eps: float = 1e-6,
    use_swizzle: bool = True,
    use_pdl: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """RMSNorm fused with W8A8-MXFP8 quantisation.

    Computes ``y = bf16(x * rsqrt(mean(x^2) + eps) * weight)`` in fp32 and
    quantises it exactly as ``group_wise_quant(y, "w8a8-mxfp8", use_swizzle)``
    does, reading ``x`` once.

    Args:
        input: [M, K] bfloat16 CUDA tensor, rows may be strided (``stride(1) == 1``,
            16-byte aligned row starts); K a multiple of 128 and at most 8192.
        weight: [K] bfloat16 RMSNorm gamma.
        eps: RMSNorm epsilon.
        use_swizzle: scales in the SfAtom layout (padding rows zero) or row-major.
        use_pdl: launch with programmatic stream serialisation.

    Returns:
        ``(q, sf)``: [M, K] float8_e4m3fn and uint8 UE8M0 scales,
        [ceil(M/128)*128, K/32] (SfAtom order) or [M, K/32] (row-major).
    """
    _check(input.dim() == 2 and input.dtype == torch.bfloat16, "input must be a 2D bfloat16 tensor [M, K]")
    m, k = input.shape
    _check(
        input.stride(1) == 1 and (input.stride(0) * 2) % 16 == 0 and input.data_ptr() % 16 == 0,
        "input rows must be contiguous and 16-byte aligned",
    )
    if not (k % 128 == 0 and 0 < k <= 8192):
        raise RuntimeError(f"K must be a multiple of 128 and at most 8192, got {k}")
    _check(
        weight.dim() == 1 and weight.size(0) == k and weight.dtype == torch.bfloat16 and weight.is_contiguous(),
        "weight must be a contiguous bfloat16 [K] tensor",
    )
    _check(input.is_cuda and weight.is_cuda, "input and weight must be CUDA tensors (this library has no CPU path)")
    m_sf = (m + 127) // 128 * 128 if use_swizzle else m
    q = torch.empty([m, k], dtype=torch.float8_e4m3fn, device=input.device)
    sf = torch.empty([m_sf, k // 32], dtype=torch.uint8, device=input.device)
    _native.call(
        "hq_rms_norm_quant",
        input.data_ptr(), input.stride(0), weight.data_ptr(), float(eps), m, k, int(bool(use_swizzle)),
        int(bool(use_pdl)), q.data_ptr(), sf.data_ptr(), input.device.index,
        _native.current_stream(input.device),
    )
    return q, sf
