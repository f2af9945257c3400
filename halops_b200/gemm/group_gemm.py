"""``group_masked_gemm`` and ``group_contiguous_gemm``: same signatures, defaults and
error texts as the reference's MoE grouped GEMMs
(``halops/gemm/group_masked_gemm.py:25-116``, ``halops/gemm/group_contiguous_gemm.py:25-105``;
host checks of ``csrc/kernel/gemm/group_masked_gemm.cu:22-186`` and
``csrc/kernel/gemm/group_contiguous_gemm.cu:22-176``), executed by this package's tcgen05
kernel through the C ABI.  Built: ``w8a8-mxfp8`` (optional per-expert bias),
``w4a4-nvfp4`` (per-expert alpha), ``w4a4-mxfp4`` and ``w4a8-mxfp4`` (float8_e4m3fn
activations x packed e2m1 weights, UE8M0 scales per 32 on both)."""

from __future__ import annotations

from typing import Optional

import torch

from .. import _native

__all__ = ["group_masked_gemm", "group_contiguous_gemm"]

_MODES = ("w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4", "w4a8-mxfp4")
_MODE_IDS = dict(_native.MODE_IDS, **{"w4a8-mxfp4": 3})  # the last one is a GEMM-only mode


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _common(input, weight, sfa, sfb, bias, alpha, mode, num_experts, n):
    """Mode-dependent operand checks shared by both grouped GEMMs; returns
    ``(k, bias_ptr, alpha_ptr)``."""
    fp8 = mode == "w8a8-mxfp8"
    if mode == "w4a8-mxfp4":
        k = weight.size(2) * 2
        _check(input.size(1) == k,
               f"W4A8 input K (unpacked fp8) must match unpacked weight K, got input K={input.size(1)}, weight K={k}")
        _check(bias is None, "W4A8 mode does not support bias yet.")
        _check(alpha is None, "W4A8 mode does not take alpha; scales are per-group UE8M0.")
        sf_k = k // 32
        _check(sfa.size(-1) == sf_k and sfb.size(-1) == sf_k,
               f"W4A8 'w4a8-mxfp4' (UE8M0 per 32) requires SF K = {sf_k}, got sfa K={sfa.size(-1)} and "
               f"sfb K={sfb.size(-1)}.")
    elif fp8:
        k = weight.size(2)
        _check(input.size(1) == k, f"input K must match weight K, got input K={input.size(1)}, weight K={k}")
    else:
        k = weight.size(2) * 2
        _check(
            input.size(1) == weight.size(2),
            f"packed input K/2 must match packed weight K/2, got input K/2={input.size(1)}, "
            f"weight K/2={weight.size(2)}",
        )
        _check(bias is None, "W4A4 mode does not support bias yet.")
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
            "'w4a4-mxfp4' does not take alpha; the per-expert scaling factor is only used by 'w4a4-nvfp4'.",
        )
        if not mxfp4:
            _check(alpha is not None, "W4A4-nvfp4 mode requires alpha input (per-expert scaling factor).")
    return k


def _pointers(bias, alpha, fp8, num_experts, n):
    bias_ptr = None
    if bias is not None:
        _check(bias.dtype == torch.bfloat16 and bias.numel() == num_experts * n and bias.is_contiguous(),
               f"bias must be a contiguous bfloat16 [num_experts, N] tensor of {num_experts * n} elements")
        _check(bias.is_cuda, "bias must be a CUDA tensor (this library has no CPU path)")
        bias_ptr = bias.data_ptr()
    alpha_ptr = None
    if alpha is not None and not fp8:
        _check(alpha.is_cuda and alpha.dtype == torch.float32 and alpha.numel() == num_experts
               and alpha.is_contiguous(), "alpha must be a float32 CUDA tensor with shape [num_experts]")
        alpha_ptr = alpha.data_ptr()
    return bias_ptr, alpha_ptr


def group_masked_gemm(
    input: torch.Tensor,
    weight: torch.Tensor,
    sfa: torch.Tensor,
    sfb: torch.Tensor,
    masked_m: torch.Tensor,
    output: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    alpha: Optional[torch.Tensor] = None,
    max_m_per_expert: int = 0,
    sm_count: int = -1,
    mode: str = "w8a8-mxfp8",
) -> None:
    """Masked grouped GEMM: expert ``e`` owns rows ``[e * max_m, (e + 1) * max_m)`` of
    ``input`` and ``output``; the first ``masked_m[e]`` of them are multiplied by
    ``weight[e]^T`` (times ``alpha[e]``, plus ``bias[e]``), the rest are left untouched.

    Args:
        input: [num_experts * max_m_per_expert, K] float8_e4m3fn, or [.., K/2] uint8 (w4a4).
        weight: [num_experts, N, K] / [num_experts, N, K/2].
        sfa: uint8 SfAtom scales over all rows of ``input``.
        sfb: uint8 SfAtom scales per expert, [num_experts, N, sf_k] (N a multiple of 128).
        masked_m: [num_experts] int32 CUDA tensor, valid rows per expert.
        output: [num_experts * max_m_per_expert, N] bfloat16, written in place.
        bias: optional [num_experts, N] bfloat16, ``w8a8-mxfp8`` only.
        alpha: float32 [num_experts]; required for ``w4a4-nvfp4``, rejected for ``w4a4-mxfp4``.
        max_m_per_expert: rows per expert slot, a positive multiple of 64.
    """
    _check(
        mode in _MODES,
        f"Unsupported mode: {mode}. Expected 'w8a8-mxfp8', 'w4a4-nvfp4', 'w4a4-mxfp4' or 'w4a8-mxfp4'.",
    )
    _check(input.dim() == 2, "input must be a 2D tensor of shape [num_experts * max_m_per_expert, K]")
    _check(weight.dim() == 3, "weight must be a 3D tensor of shape [num_experts, N, K]")
    _check(masked_m.dim() == 1, "masked_m must be a 1D tensor of shape [num_experts]")
    _check(masked_m.dtype == torch.int32, "masked_m must have dtype torch.int32")
    _check(output.dim() == 2, "output must be a 2D tensor of shape [M, N]")
    _check(max_m_per_expert > 0, f"max_m_per_expert must be greater than 0, got {max_m_per_expert}")
    m, n, num_experts = input.size(0), weight.size(1), weight.size(0)
    _check(masked_m.size(0) == num_experts,
           f"masked_m shape must be [num_experts], got {masked_m.size(0)}, expected {num_experts}")
    _check(m == num_experts * max_m_per_expert,
           f"input M must equal num_experts * max_m_per_expert, got {m}, expected {num_experts * max_m_per_expert}")
    _check(output.size(0) == m and output.size(1) == n,
           f"output shape must be [M, N], got [{output.size(0)}, {output.size(1)}], expected [{m}, {n}]")
    k = _common(input, weight, sfa, sfb, bias, alpha, mode, num_experts, n)
    _check(output.dtype == torch.bfloat16, "output must be a bfloat16 tensor")
    _check(input.is_contiguous() and weight.is_contiguous() and sfa.is_contiguous() and sfb.is_contiguous()
           and masked_m.is_contiguous(), "input, weight, sfa, sfb and masked_m must be contiguous")
    _check(output.stride(1) == 1, "output rows must be contiguous")
    if m == 0 or n == 0:
        return
    _native.call("hq_describe_group_tile", 2, num_experts, max_m_per_expert, m, n, k, _MODE_IDS[mode], 148, -1)
    bias_ptr, alpha_ptr = _pointers(bias, alpha, mode == "w8a8-mxfp8", num_experts, n)
    for name, t in (("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("masked_m", masked_m),
                    ("output", output)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor (this library has no CPU path)")
    _native.call(
        "hq_group_masked_gemm",
        input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), masked_m.data_ptr(), output.data_ptr(),
        bias_ptr, alpha_ptr, num_experts, max_m_per_expert, n, k, sfa.numel(), sfb.numel(), output.stride(0),
        _MODE_IDS[mode], int(sm_count), 1, input.device.index,
        _native.current_stream(input.device),
    )


def group_contiguous_gemm(
    input: torch.Tensor,
    weight: torch.Tensor,
    sfa: torch.Tensor,
    sfb: torch.Tensor,
    expert_ids: torch.Tensor,
    output: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    alpha: Optional[torch.Tensor] = None,
    sm_count: int = -1,
    mode: str = "w8a8-mxfp8",
) -> None:
    """Contiguous grouped GEMM: row ``r`` of ``input`` is multiplied by
    ``weight[expert_ids[r]]^T`` (times ``alpha[e]``, plus ``bias[e]``).

    Args:
        input: [M, K] float8_e4m3fn, or [M, K/2] uint8 (w4a4); M a multiple of 64.
        weight: [num_experts, N, K] / [num_experts, N, K/2].
        sfa: uint8 SfAtom scales over the rows of ``input``.
        sfb: uint8 SfAtom scales per expert, [num_experts, N, sf_k] (N a multiple of 128).
        expert_ids: [M] int32 CUDA tensor, non-decreasing; every run of equal ids
            starts on a multiple of 64 rows.
        output: [M, N] bfloat16, written in place.
        bias / alpha: per expert, as for ``group_masked_gemm``.
    """
    _check(
        mode in _MODES,
        f"Unsupported mode: {mode}. Expected 'w8a8-mxfp8', 'w4a4-nvfp4', 'w4a4-mxfp4' or 'w4a8-mxfp4'.",
    )
    _check(input.dim() == 2, "input must be a 2D tensor of shape [M, K]")
    _check(weight.dim() == 3, "weight must be a 3D tensor of shape [num_experts, N, K]")
    _check(expert_ids.dim() == 1, "expert_ids must be a 1D tensor of shape [M]")
    _check(expert_ids.dtype == torch.int32, "expert_ids must have dtype torch.int32")
    _check(output.dim() == 2, "output must be a 2D tensor of shape [M, N]")
    m, n, num_experts = input.size(0), weight.size(1), weight.size(0)
    _check(expert_ids.size(0) == m, f"expert_ids shape must be [M], got {expert_ids.size(0)}, expected {m}")
    _check(output.size(0) == m and output.size(1) == n,
           f"output shape must be [M, N], got [{output.size(0)}, {output.size(1)}], expected [{m}, {n}]")
    k = _common(input, weight, sfa, sfb, bias, alpha, mode, num_experts, n)
    _check(output.dtype == torch.bfloat16, "output must be a bfloat16 tensor")
    _check(input.is_contiguous() and weight.is_contiguous() and sfa.is_contiguous() and sfb.is_contiguous()
           and expert_ids.is_contiguous(), "input, weight, sfa, sfb and expert_ids must be contiguous")
    _check(output.stride(1) == 1, "output rows must be contiguous")
    if m == 0 or n == 0 or num_experts == 0:
        return
    _native.call("hq_describe_group_tile", 3, num_experts, m // num_experts, m, n, k, _MODE_IDS[mode], 148, -1)
    bias_ptr, alpha_ptr = _pointers(bias, alpha, mode == "w8a8-mxfp8", num_experts, n)
    for name, t in (("input", input), ("weight", weight), ("sfa", sfa), ("sfb", sfb), ("expert_ids", expert_ids),
                    ("output", output)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor (this library has no CPU path)")
    _native.call(
        "hq_group_contiguous_gemm",
        input.data_ptr(), weight.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), expert_ids.data_ptr(),
        output.data_ptr(), bias_ptr, alpha_ptr, num_experts, m, n, k, sfa.numel(), sfb.numel(), output.stride(0),
        _MODE_IDS[mode], int(sm_count), 1, input.device.index,
        _native.current_stream(input.device),
    )
