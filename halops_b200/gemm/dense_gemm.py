"""``dense_gemm``: same signature, defaults and error texts as the reference's
``halops.dense_gemm`` (``halops/gemm/dense_gemm.py:44-135``; host checks of
``csrc/kernel/gemm/dense_gemm.cu:23-189``), executed by this package's
tcgen05 kernel through the C ABI.  Built: the Identity and Sigmoid epilogues
for ``w8a8-mxfp8``, ``w4a4-nvfp4`` and ``w4a4-mxfp4``, an optional bias and the
SituQuant (SiTU-GLU + MXFP8 re-quantisation) epilogue for ``w8a8-mxfp8``."""

from __future__ import annotations

import enum
from typing import Optional

import torch

from .. import _native

__all__ = ["dense_gemm", "interleave_gate_up", "EpilogueOp"]

_GLU_INTERLEAVE = 16


class EpilogueOp(enum.IntEnum):
    """Values of the reference enum (``csrc/kernel/gemm/epilogue_op.h:21-28``)."""

    Identity = 0
    Quant = 1
    GateMulQuant = 2
    Sigmoid = 3
    SituQuant = 4
    SigmoidGateMulQuant = 5


def interleave_gate_up(t: torch.Tensor) -> torch.Tensor:
    """Reorder ``[gate; up]`` rows into alternating blocks of 16 rows (gate rows
    ``16i..16i+15``, then up rows ``16i..16i+15``), the row order the
    reference's SituQuant epilogue expects (``halops/gemm/dense_gemm.py:30-41``)."""
    half = t.size(0) // 2
    if t.size(0) != 2 * half or half % _GLU_INTERLEAVE != 0:
        raise RuntimeError(f"interleave_gate_up needs 2 * I rows with I a multiple of {_GLU_INTERLEAVE}, "
                           f"got {t.size(0)}")
    # output block 2i is gate block i, output block 2i + 1 is up block i
    blocks = t.reshape(2, half // _GLU_INTERLEAVE, _GLU_INTERLEAVE, *t.shape[1:])
    return blocks.transpose(0, 1).reshape(t.shape)


# dense shapes that hq_describe_tile has accepted (the check does not depend on the device)
_LEGAL_SHAPES: set = set()


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def dense_gemm(
    input: torch.Tensor,
    weight: torch.Tensor,
    sfa: torch.Tensor,
    sfb: torch.Tensor,
    output: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    alpha: Optional[torch.Tensor] = None,
    sm_count: int = -1,
    mode: str = "w8a8-mxfp8",
    use_pdl: bool = True,
    epilogue: EpilogueOp = EpilogueOp.Identity,
    output_sf: Optional[torch.Tensor] = None,
    situ_beta: float = 4.0,
    situ_linear_beta: Optional[float] = 25.0,
) -> None:
    """``output = bf16(alpha * (input @ weight^T))`` on the sm_100a tensor cores.

    Args:
        input: [M, K] float8_e4m3fn, or [M, K/2] uint8 packed e2m1 (w4a4 modes).
        weight: [N, K] / [N, K/2], same encoding.
        sfa / sfb: uint8 block scales in SfAtom order covering whole 128-row
            atoms, exactly what ``group_wise_quant`` returns.
        output: [M, N] bfloat16, written in place.
        alpha: float32 [1]; required for ``w4a4-nvfp4``, rejected for
            ``w4a4-mxfp4``, ignored for ``w8a8-mxfp8``.
        sm_count: SMs to use (-1: all).
        mode: ``"w8a8-mxfp8"``, ``"w4a4-mxfp4"`` or ``"w4a4-nvfp4"``.
        use_pdl: launch with programmatic stream serialisation.  ``2`` (not in the reference) adds the
            promise that ``weight`` and ``sfb`` are not written by the kernel that precedes this call on
            the stream; the small-M kernel then streams the weight of its first stages while that kernel
            is still finishing (chains of decode GEMMs).
        bias: optional [N] bfloat16 vector, ``w8a8-mxfp8`` only, M a multiple of 256
            (the reference's rule).
        epilogue: what happens to ``y = alpha * input @ weight^T + bias`` before it is stored.
            ``EpilogueOp.Identity`` stores ``bf16(y)``; ``EpilogueOp.Sigmoid`` stores
            ``bf16(sigmoid(y))``.  ``EpilogueOp.SituQuant`` (``w8a8-mxfp8`` only) is the fused
            SiTU-GLU activation plus re-quantisation: the weight holds a gate and an up
            projection whose rows (and those of sfb and bias) were put in
            ``interleave_gate_up`` order, so every 32 accumulator columns carry 16 gate
            values ``g`` and the 16 matching up values ``u``.  The kernel forms
            ``z = situ_beta * tanh(g / situ_beta) * sigmoid(g) * c(u)`` with
            ``c(u) = situ_linear_beta * tanh(u / situ_linear_beta)``, or ``c(u) = u`` when
            ``situ_linear_beta`` is None, and writes ``z`` as MXFP8: ``output`` is then
            ``[M, N/2]`` float8_e4m3fn and ``output_sf`` receives one UE8M0 scale per 32
            output columns.
        output_sf: SfAtom scales of the quantised output ([ceil(M/128)*128, N/64] uint8).
        situ_beta / situ_linear_beta: gate and up soft-caps.
    """
    # (the messages are only built when a check fails: this function runs once per GEMM of a
    # decode step, where the host's time per call is what the step costs)
    if mode not in _native.MODE_IDS:
        raise RuntimeError(f"Unsupported mode: {mode}. Expected 'w8a8-mxfp8', 'w4a4-mxfp4' or 'w4a4-nvfp4'.")
    if input.dim() != 2:
        raise RuntimeError("input must be a 2D tensor of shape [M, K]")
    if weight.dim() != 2:
        raise RuntimeError("weight must be a 2D tensor of shape [N, K]")
    if output.dim() != 2:
        raise RuntimeError("output must be a 2D tensor of shape [M, N]")
    epilogue = EpilogueOp(int(epilogue))
    m, in_k = input.shape
    n, w_k = weight.shape
    out_m, out_cols = output.shape
    out_n = n // 2 if epilogue == EpilogueOp.SituQuant else n
    if out_m != m or out_cols != out_n:
        raise RuntimeError(f"output shape must be [{m}, {out_n}], got [{out_m}, {out_cols}]")
    m_sf = (m + 127) // 128 * 128
    fp8 = mode == "w8a8-mxfp8"
    if fp8:
        k = w_k
        if in_k != k:
            raise RuntimeError(f"input K must match weight K, got input K={in_k}, weight K={k}")
        if sfb.dtype != torch.uint8:
            raise RuntimeError("sfb must be the uint8 SfAtom weight scale that group_wise_quant returns")
        sf_k = k // 32
        if not (sfa.is_contiguous() and sfa.numel() >= m_sf * sf_k):
            raise RuntimeError(f"sfa must hold whole 128-row SfAtoms: expected at least {m_sf * sf_k} elements "
                               f"({m_sf} x {sf_k}) for M={m}, got {sfa.numel()}")
        if bias is not None and epilogue != EpilogueOp.SituQuant and m % 256 != 0:
            raise RuntimeError("the bias tile has no per-row store predicate yet, so M must be a multiple of 256 "
                               f"when bias is given, got {m}")
    else:
        k = w_k * 2
        if in_k != w_k:
            raise RuntimeError(f"packed input K/2 must match packed weight K/2, got input K/2={in_k}, "
                               f"weight K/2={w_k}")
        if bias is not None:
            raise RuntimeError("W4A4 mode does not support bias yet.")
        mxfp4 = mode == "w4a4-mxfp4"
        if mxfp4 and alpha is not None:
            raise RuntimeError(
                "'w4a4-mxfp4' does not take alpha; the global scaling factor is only used by 'w4a4-nvfp4'.")
        sf_k = k // (32 if mxfp4 else 16)
        if sfa.size(-1) != sf_k or sfb.size(-1) != sf_k:
            raise RuntimeError(
                "W4A4 scale-factor shape does not match mode "
                + ("'w4a4-mxfp4' (UE8M0 per 32)" if mxfp4 else "'w4a4-nvfp4' (UE4M3 per 16)")
                + f" requires SF K = {sf_k}, got sfa K={sfa.size(-1)} and sfb K={sfb.size(-1)}.")
        if not (sfa.is_contiguous() and sfa.numel() >= m_sf * sf_k):
            raise RuntimeError(f"sfa must hold whole 128-row SfAtoms: expected at least {m_sf * sf_k} elements "
                               f"({m_sf} x {sf_k}) for M={m}, got {sfa.numel()}")
        if not mxfp4 and alpha is None:
            raise RuntimeError("W4A4-nvfp4 mode requires alpha input (per-batch scaling).")
    if not (epilogue in (EpilogueOp.Identity, EpilogueOp.Sigmoid) or (epilogue == EpilogueOp.SituQuant and fp8)):
        raise RuntimeError(f"Unsupported epilogue {int(epilogue)} for {mode}")
    bias_ptr = None
    if bias is not None:
        _check(bias.dtype == torch.bfloat16 and bias.dim() == 1 and bias.numel() == n and bias.is_contiguous(),
               f"bias must be a contiguous bfloat16 vector of {n} elements")
        _check(bias.is_cuda, "bias must be a CUDA tensor (this library has no CPU path)")
        bias_ptr = bias.data_ptr()
    if epilogue == EpilogueOp.SituQuant:
        _check(output.dtype == torch.float8_e4m3fn and output.is_contiguous(),
               "output must be a contiguous float8_e4m3fn tensor for EpilogueOp.SituQuant")
        _check(output_sf is not None and output_sf.dtype == torch.uint8 and output_sf.is_contiguous(),
               "EpilogueOp.SituQuant needs a contiguous uint8 output_sf")
        _check(input.is_contiguous() and weight.is_contiguous() and sfb.is_contiguous(),
               "input, weight and sfb must be contiguous")
        if m > 0 and n > 0:
            _native.call("hq_describe_tile", m, n, k, _native.MODE_IDS[mode], 148, -1)
        for name, t in (("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("output", output),
                        ("output_sf", output_sf)):
            _check(t.is_cuda, f"{name} must be a CUDA tensor (this library has no CPU path)")
        _native.call(
            "hq_dense_gemm_situ_quant",
            input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), output.data_ptr(),
            output_sf.data_ptr(), bias_ptr, m, n, k, sfa.numel(), sfb.numel(), output_sf.numel(),
            float(situ_beta), 0.0 if situ_linear_beta is None else float(situ_linear_beta), int(sm_count),
            int(bool(use_pdl)), input.device.index, _native.current_stream(input.device),
        )
        return
    _check(output.dtype == torch.bfloat16, "output must be a bfloat16 tensor")
    _check(input.is_contiguous() and weight.is_contiguous() and sfb.is_contiguous(),
           "input, weight and sfb must be contiguous")
    _check(output.stride(1) == 1, "output rows must be contiguous")
    if m > 0 and n > 0 and (m, n, k, mode) not in _LEGAL_SHAPES:
        # shape legality ("No dense ... tile") is reported before anything touches a device
        _native.call("hq_describe_tile", m, n, k, _native.MODE_IDS[mode], 148, -1)
        if len(_LEGAL_SHAPES) < 4096:
            _LEGAL_SHAPES.add((m, n, k, mode))
    alpha_ptr = None
    if alpha is not None and not fp8:
        _check(alpha.is_cuda and alpha.dtype == torch.float32 and alpha.numel() >= 1,
               "alpha must be a float32 CUDA tensor with shape [1]")
        alpha_ptr = alpha.data_ptr()
    for name, t in (("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("output", output)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor (this library has no CPU path)")
    dev = input.device.index
    stream = _native.current_stream(input.device)
    _native.call(
        "hq_dense_gemm",
        input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), output.data_ptr(), bias_ptr, alpha_ptr,
        m, n, k, sfa.numel(), sfb.numel(), output.stride(0) if m > 0 else max(n, 8),
        _native.MODE_IDS[mode], int(epilogue), int(sm_count), 2 if use_pdl == 2 else int(bool(use_pdl)), dev, stream,
    )
