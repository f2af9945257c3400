"""``group_wise_quant``: same signature, defaults, shapes, dtypes and error
texts as the reference's ``halops.group_wise_quant``
(``halops/gemm/group_wise_quant.py:26-84``; host checks of
``csrc/kernel/gemm/group_wise_quant.cu:297-375``), executed by this package's
sm_100a kernel through the C ABI."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native

__all__ = ["group_wise_quant"]

_DTYPE_IDS = {torch.bfloat16: 0, torch.float16: 1}


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def group_wise_quant(
    input: torch.Tensor,
    mode: str = "w8a8-mxfp8",
    use_swizzle: bool = True,
    use_pdl: bool = True,
    output_quant: Optional[torch.Tensor] = None,
    output_sf: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-wise quantisation from BF16/FP16 to FP8/FP4 with block scales.

    Args:
        input: [m, k] CUDA tensor, bfloat16 or float16; rows may be strided
            (``stride(1) == 1``, 16-byte aligned row starts).
        mode: ``"w8a8-mxfp8"`` (e4m3, UE8M0 per 32), ``"w4a4-mxfp4"`` (packed
            e2m1, UE8M0 per 32) or ``"w4a4-nvfp4"`` (packed e2m1, UE4M3 per 16).
        use_swizzle: scales in the 128x4 SfAtom order the GEMM consumes
            (rows padded to a multiple of 128, padding zero) or row-major.
        use_pdl: launch with programmatic stream serialisation.
        output_quant / output_sf: optional pre-allocated contiguous outputs,
            returned as they are.

    Returns:
        ``(output_quant, output_sf)``: [m, k] float8_e4m3fn or [m, k/2] uint8,
        and [ceil(m/128)*128 or m, k / group] uint8.
    """
    # (the messages are only built when a check fails: this runs once per activation of a decode step)
    if input.dim() != 2:
        raise RuntimeError("input must be a 2D tensor of shape [m, k]")
    if input.dtype not in _DTYPE_IDS:
        raise RuntimeError("input dtype must be bfloat16 or float16")
    if not (input.stride(1) == 1 and (input.stride(0) * 2) % 16 == 0 and input.data_ptr() % 16 == 0):
        raise RuntimeError("input rows must be contiguous and 16-byte aligned")
    if mode not in _native.MODE_IDS:
        raise RuntimeError(
            f"Unsupported quantization mode: {mode}. Expected 'w8a8-mxfp8', 'w4a4-mxfp4' or 'w4a4-nvfp4'.")
    group = _native.GROUP_SIZE[mode]
    m, k = input.shape
    kb_dim = k // group
    if k % group != 0:
        raise RuntimeError(f"k must be divisible by the quantization group size ({group}) for mode {mode}, got k={k}")
    if use_swizzle and kb_dim % 4 != 0:
        raise RuntimeError(f"scale kb_dim must be divisible by 4 for CUTLASS SfAtom layout, got {kb_dim}")
    m_sf = (m + 127) // 128 * 128 if use_swizzle else m
    fp4 = mode != "w8a8-mxfp8"
    quant_dtype = torch.uint8 if fp4 else torch.float8_e4m3fn
    quant_k = k // 2 if fp4 else k
    if output_quant is None:
        output_quant = torch.empty([m, quant_k], dtype=quant_dtype, device=input.device)
    elif not (output_quant.is_contiguous() and output_quant.dtype == quant_dtype
              and output_quant.numel() == m * quant_k and output_quant.device == input.device):
        raise RuntimeError(f"output_quant must be a contiguous [{m}, {quant_k}] tensor of the mode's dtype")
    if output_sf is None:
        output_sf = torch.empty([m_sf, kb_dim], dtype=torch.uint8, device=input.device)
    elif not (output_sf.is_contiguous() and output_sf.dtype == torch.uint8
              and output_sf.numel() == m_sf * kb_dim and output_sf.device == input.device):
        raise RuntimeError(f"output_sf must be a contiguous uint8 tensor of {m_sf} x {kb_dim} elements")
    _check(input.is_cuda, "input must be a CUDA tensor (this library has no CPU path)")
    dev = input.device.index
    stream = _native.current_stream(input.device)
    _native.call(
        "hq_group_wise_quant",
        input.data_ptr(), input.stride(0), _DTYPE_IDS[input.dtype], m, k, _native.MODE_IDS[mode],
        int(bool(use_swizzle)), int(bool(use_pdl)), output_quant.data_ptr(), output_sf.data_ptr(),
        dev, stream,
    )
    return output_quant, output_sf
