"""``batch_gemm``: same signature, defaults and error texts as the reference's
``halops.batch_gemm`` (``halops/gemm/batch_gemm.py:27-117``; host checks of
``csrc/kernel/gemm/batch_gemm.cu:22-188``), executed by this package's tcgen05
kernel through the C ABI.  Built: the Identity epilogue for ``w8a8-mxfp8``
(optional per-batch bias), ``w4a4-nvfp4`` (per-batch alpha) and ``w4a4-mxfp4``, and the
quantising epilogues (Quant, GateMulQuant, SigmoidGateMulQuant) for ``w8a8-mxfp8``."""

from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from .dense_gemm import EpilogueOp

__all__ = ["batch_gemm"]


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def batch_gemm(
    input: torch.Tensor,
    weight: torch.Tensor,
    sfa: torch.Tensor,
    sfb: torch.Tensor,
    output: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    alpha: Optional[torch.Tensor] = None,
    sm_count: int = -1,
    mode: str = "w8a8-mxfp8",
    epilogue: EpilogueOp = EpilogueOp.Identity,
    output_sf: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
    use_pdl: bool = True,
) -> None:
    """``output[:, b*N:(b+1)*N] = bf16(alpha[b] * (input[b] @ weight[b]^T) + bias[b])``.

    Args:
        input: [B, M, K] float8_e4m3fn, or [B, M, K/2] uint8 packed e2m1 (w4a4 modes).
        weight: [B, N, K] / [B, N, K/2], same encoding.
        sfa: uint8 SfAtom scales over the stacked rows, ``[ceil(B*M/128)*128, sf_k]``
            (``group_wise_quant`` of the ``[B*M, K]`` view).
        sfb: uint8 SfAtom scales per batch, ``[B, N, sf_k]`` with N a multiple of 128
            (``[B, ceil(N/128)*128, sf_k]`` otherwise).
        output: [M, B*N] bfloat16 (float8_e4m3fn for the quantising epilogues), written in
            place; rows may be strided.
        bias: optional [B, N] bfloat16, ``w8a8-mxfp8`` only.
        alpha: float32 [B]; required for ``w4a4-nvfp4``, rejected for ``w4a4-mxfp4``,
            ignored for ``w8a8-mxfp8``.
        sm_count: SMs to use (-1: all).
        epilogue: ``EpilogueOp.Identity``, or for ``w8a8-mxfp8`` ``EpilogueOp.Quant``,
            ``EpilogueOp.GateMulQuant`` or ``EpilogueOp.SigmoidGateMulQuant``: the bfloat16 result
            (times ``gate``, or times ``bf16(sigmoid(gate))``) re-quantised to MXFP8 per 32 columns.
        output_sf: UE8M0 SfAtom scales of the quantised output over ``[M, B*N/32]``
            (``ceil(M/128)*128 * B*N/32`` bytes; N a multiple of 128).
        gate: [M, B*N] bfloat16 (logits for the sigmoid form); rows may be strided
            (``stride(1) == 1``, 32-byte aligned row starts).
        use_pdl: launch with programmatic stream serialisation.
    """
    _check(
        mode in _native.MODE_IDS,
        f"Unsupported mode: {mode}. Expected 'w8a8-mxfp8', 'w4a4-nvfp4' or 'w4a4-mxfp4'.",
    )
    _check(input.dim() == 3, "input must be a 3D tensor of shape [B, M, K]")
    _check(weight.dim() == 3, "weight must be a 3D tensor of shape [B, N, K]")
    _check(output.dim() == 2, "output must be a 2D tensor of shape [M, B * N]")
    batches, m, n = input.size(0), input.size(1), weight.size(1)
    _check(weight.size(0) == batches, f"weight batch dim must match input batch dim, got {weight.size(0)}")
    _check(output.size(0) == m and output.size(1) == batches * n, "output shape must be [M, B * N]")
    _check(output_sf is None or n % 128 == 0, f"quantized output needs N % 128 == 0, got {n}")
    epilogue = EpilogueOp(int(epilogue))
    fp8 = mode == "w8a8-mxfp8"
    if fp8:
        k = weight.size(2)
        _check(input.size(2) == k, f"input K must match weight K, got input K={input.size(2)}, weight K={k}")
        _check(gate is not None or epilogue not in (EpilogueOp.GateMulQuant, EpilogueOp.SigmoidGateMulQuant),
               "GateMulQuant epilogues need gate")
        sf_k = k // 32
    else:
        k = weight.size(2) * 2
        _check(
            input.size(2) == weight.size(2),
            f"packed input K/2 must match packed weight K/2, got {input.size(2)}, weight K/2={weight.size(2)}",
        )
        _check(bias is None, "W4A4 batch GEMM does not support bias yet.")
        mxfp4 = mode == "w4a4-mxfp4"
        sf_k = k // (32 if mxfp4 else 16)
        _check(
            sfa.size(-1) == sf_k and sfb.size(-1) == sf_k,
            "W4A4 scale-factor shape does not match mode "
            + ("'w4a4-mxfp4' (UE8M0 per 32)" if mxfp4 else "'w4a4-nvfp4' (UE4M3 per 16)")
            + f" requires SF K = {sf_k}, got sfa K={sfa.size(-1)} and sfb K={sfb.size(-1)}.",
        )
        _check(
            not mxfp4 or alpha is None,
            "'w4a4-mxfp4' does not take alpha; the per-batch scaling factor is only used by 'w4a4-nvfp4'.",
        )
        if not mxfp4:
            _check(alpha is not None, "W4A4-nvfp4 mode requires alpha input (per-batch scaling).")
    quant_ops = (EpilogueOp.Quant, EpilogueOp.GateMulQuant, EpilogueOp.SigmoidGateMulQuant)
    _check(epilogue == EpilogueOp.Identity or (fp8 and epilogue in quant_ops),
           f"Unsupported epilogue {int(epilogue)} for {mode}")
    if epilogue in quant_ops:
        _check(n % 128 == 0, f"quantized output needs N % 128 == 0, got {n}")
        _check(output.dtype == torch.float8_e4m3fn and output.stride(1) == 1,
               "output must be a float8_e4m3fn tensor with contiguous rows for the quantising epilogues")
        _check(output_sf is not None and output_sf.dtype == torch.uint8 and output_sf.is_contiguous(),
               "the quantising epilogues need a contiguous uint8 output_sf")
        gate_ptr, gate_ld = None, 0
        if epilogue != EpilogueOp.Quant:
            _check(gate.dtype == torch.bfloat16 and tuple(gate.shape) == tuple(output.shape),
                   "gate must be a bfloat16 [M, B * N] tensor")
            _check(gate.stride(1) == 1 and gate.stride(0) * 2 % 32 == 0 and gate.data_ptr() % 32 == 0,
                   "gate rows must be contiguous and 32-byte aligned")
            gate_ptr, gate_ld = gate.data_ptr(), gate.stride(0)
        _check(input.is_contiguous() and weight.is_contiguous() and sfa.is_contiguous() and sfb.is_contiguous(),
               "input, weight, sfa and sfb must be contiguous")
        if batches == 0 or m == 0 or n == 0:
            return
        _native.call("hq_describe_group_tile", 1, batches, m, batches * m, n, k, _native.MODE_IDS[mode], 148, -1)
        bias_ptr = None
        if bias is not None:
            _check(bias.dtype == torch.bfloat16 and bias.numel() == batches * n and bias.is_contiguous(),
                   f"bias must be a contiguous bfloat16 [B, N] tensor of {batches * n} elements")
            bias_ptr = bias.data_ptr()
        tensors = [("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("output", output),
                   ("output_sf", output_sf)] + ([("gate", gate)] if gate_ptr else []) \
            + ([("bias", bias)] if bias is not None else [])
        for name, t in tensors:
            _check(t.is_cuda, f"{name} must be a CUDA tensor (this library has no CPU path)")
        _native.call(
            "hq_batch_gemm_quant",
            input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), output.data_ptr(),
            output_sf.data_ptr(), gate_ptr, gate_ld, bias_ptr, batches, m, n, k, sfa.numel(), sfb.numel(),
            output.stride(0), output_sf.numel(), int(epilogue), int(sm_count), int(bool(use_pdl)),
            input.device.index, _native.current_stream(input.device),
        )
        return
    _check(output_sf is None and gate is None, "output_sf and gate belong to the quantising epilogues")
    _check(output.dtype == torch.bfloat16, "output must be a bfloat16 tensor")
    _check(input.is_contiguous() and weight.is_contiguous() and sfa.is_contiguous() and sfb.is_contiguous(),
           "input, weight, sfa and sfb must be contiguous")
    _check(output.stride(1) == 1, "output rows must be contiguous")
    if batches == 0 or m == 0 or n == 0:
        return
    # shape legality ("No batch ... tile") is reported before anything touches a device
    _native.call("hq_describe_group_tile", 1, batches, m, batches * m, n, k, _native.MODE_IDS[mode], 148, -1)
    bias_ptr = None
    if bias is not None:
        _check(bias.dtype == torch.bfloat16 and bias.numel() == batches * n and bias.is_contiguous(),
               f"bias must be a contiguous bfloat16 [B, N] tensor of {batches * n} elements")
        _check(bias.is_cuda, "bias must be a CUDA tensor (this library has no CPU path)")
        bias_ptr = bias.data_ptr()
    alpha_ptr = None
    if alpha is not None and not fp8:
        _check(alpha.is_cuda and alpha.dtype == torch.float32 and alpha.numel() == batches
               and alpha.is_contiguous(), "alpha must be a float32 CUDA tensor with shape [B]")
        alpha_ptr = alpha.data_ptr()
    for name, t in (("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("output", output)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor (this library has no CPU path)")
    _native.call(
        "hq_batch_gemm",
        input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), output.data_ptr(), bias_ptr, alpha_ptr,
        batches, m, n, k, sfa.numel(), sfb.numel(), output.stride(0),
        _native.MODE_IDS[mode], int(epilogue), int(sm_count), int(bool(use_pdl)), input.device.index,
        _native.current_stream(input.device),
    )
