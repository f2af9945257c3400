"""CPU restatement of the reference's dequantise-then-matmul GEMM check.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows the reference's ``tests/test_dense_gemm.py:48-74`` (``ref_gemm`` /
``ref_gemm_w4a4``): both operands are expanded to float32 with their block
scales, multiplied with ``torch.matmul`` in float32 and rounded to bfloat16.
The scale decoders follow ``tests/utils/gemm_utils.py:68-71,247-254``.  The
optional ``alpha`` is the per-tensor factor the NVFP4 kernel applies to the
float32 accumulator before the bfloat16 rounding
(``csrc/kernel/gemm/dense_gemm.cu:159-164``).
"""

from __future__ import annotations

import numpy as np
import torch

from .quant import (
    GROUP_SIZE,
    decode_e2m1_packed,
    decode_e4m3,
    decode_ue4m3,
    decode_ue8m0,
    unswizzle_sf,
)


def _np(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().to("cpu")
        if x.dtype != torch.uint8:
            x = x.view(torch.uint8)
        return x.numpy()
    return np.asarray(x, dtype=np.uint8)


def dequantize(q, sf, mode: str, rows: int | None = None, swizzled: bool = True) -> torch.Tensor:
    """Quantised bytes + block scales -> float32 [rows, k] tensor."""
    q = _np(q)
    sf = _np(sf)
    g = GROUP_SIZE[mode]
    rows = q.shape[0] if rows is None else rows
    vals = decode_e4m3(q) if mode == "w8a8-mxfp8" else decode_e2m1_packed(q)
    k = vals.shape[1]
    sf = sf.reshape(-1, k // g)
    sf_logical = unswizzle_sf(sf, rows) if swizzled else sf[:rows]
    scale = decode_ue4m3(sf_logical) if mode == "w4a4-nvfp4" else decode_ue8m0(sf_logical)
    return torch.from_numpy(vals[:rows] * np.repeat(scale, g, axis=1))


def dense_gemm_ref(a_q, b_q, sfa, sfb, mode: str = "w8a8-mxfp8", alpha: float | None = None,
                   swizzled: bool = True, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``bf16(alpha * (dequant(A) @ dequant(B)^T))`` in float32 on the CPU.

    ``a_q`` [M, K or K/2], ``b_q`` [N, K or K/2]; ``sfa`` / ``sfb`` in SfAtom
    order when ``swizzled`` (what the GEMM kernel consumes) else logical.
    Pass ``out_dtype=torch.float32`` to skip the final rounding."""
    a = dequantize(a_q, sfa, mode, swizzled=swizzled)
    b = dequantize(b_q, sfb, mode, swizzled=swizzled)
    acc = torch.matmul(a, b.T)
    if alpha is not None:
        acc = acc * float(alpha)
    return acc.to(out_dtype)


def batch_gemm_ref(a_q, b_q, sfa, sfb, mode: str = "w8a8-mxfp8", alpha=None, bias=None,
                   out_dtype=torch.bfloat16) -> torch.Tensor:
    """``out[:, b*N:(b+1)*N] = alpha[b] * (dequant(A[b]) @ dequant(B[b])^T) + bias[b]``.

    Follows the reference's ``tests/test_batch_gemm.py:49-100`` (``ref_batch_gemm_fp8`` /
    ``ref_batch_gemm_fp4``) and the token-major output of ``assert_close_per_batch``
    there: ``a_q`` [B, M, K or K/2] with ``sfa`` in SfAtom order over the stacked
    ``B * M`` rows, ``b_q`` [B, N, K or K/2] with ``sfb`` in SfAtom order per batch.
    As in the reference model, the product is rounded to bfloat16 first and the bias is
    added to that in bfloat16 arithmetic; with ``out_dtype=torch.float32`` nothing is
    rounded and the bias is added to the float32 product."""
    a_q = _np(a_q)
    b_q = _np(b_q)
    batches, m = a_q.shape[0], a_q.shape[1]
    n = b_q.shape[1]
    g = GROUP_SIZE[mode]
    k = a_q.shape[2] * (1 if mode == "w8a8-mxfp8" else 2)
    a = dequantize(a_q.reshape(batches * m, -1), sfa, mode)
    sfb = _np(sfb).reshape(batches, -1, k // g)
    out = torch.empty([m, batches * n], dtype=torch.float32)
    for b in range(batches):
        w = dequantize(b_q[b], sfb[b], mode)
        acc = torch.matmul(a[b * m:(b + 1) * m], w.T)
        if alpha is not None:
            acc = acc * float(alpha[b])
        if bias is not None:
            row = bias[b].cpu().reshape(1, n)
            if out_dtype == torch.bfloat16:
                acc = (acc.to(torch.bfloat16) + row.to(torch.bfloat16)).float()
            else:
                acc = acc + row.float()
        out[:, b * n:(b + 1) * n] = acc
    return out.to(out_dtype)


def group_gemm_ref(a_q, b_q, sfa, sfb, expert_of_row, mode: str = "w8a8-mxfp8", alpha=None, bias=None,
                   out_dtype=torch.bfloat16) -> torch.Tensor:
    """Row-wise expert GEMM: ``out[r] = alpha[e] * (dequant(A[r]) @ dequant(B[e])^T) + bias[e]``
    with ``e = expert_of_row[r]``; rows whose expert is negative stay zero.

    One model for both MoE layouts of the reference: masked
    (``tests/test_group_masked_gemm.py:88-146``: expert ``e`` owns a padded slot of which
    the first ``masked_m[e]`` rows are valid; pass -1 for the padding rows) and contiguous
    (``tests/test_group_contiguous_gemm.py:60-110``: ``expert_ids`` per row).  ``a_q``
    [M, K or K/2] with ``sfa`` in SfAtom order over its rows, ``b_q`` [E, N, K or K/2] with
    ``sfb`` in SfAtom order per expert."""
    a_q = _np(a_q)
    b_q = _np(b_q)
    experts, n = b_q.shape[0], b_q.shape[1]
    # "w4a8-mxfp4" (tests/test_group_masked_gemm.py:563-600): e4m3 activations, packed e2m1
    # weights, UE8M0 scales per 32 on both
    mode_a, mode_b = ("w8a8-mxfp8", "w4a4-mxfp4") if mode == "w4a8-mxfp4" else (mode, mode)
    g = GROUP_SIZE[mode_b]
    k = a_q.shape[1] * (1 if mode_a == "w8a8-mxfp8" else 2)
    a = dequantize(a_q, sfa, mode_a)
    mode = mode_b
    sfb = _np(sfb).reshape(experts, -1, k // g)
    ids = np.asarray(expert_of_row).astype(np.int64)
    out = torch.zeros([a_q.shape[0], n], dtype=torch.float32)
    for e in range(experts):
        rows = torch.from_numpy(np.nonzero(ids == e)[0])
        if rows.numel() == 0:
            continue
        acc = torch.matmul(a[rows], dequantize(b_q[e], sfb[e], mode).T)
        if alpha is not None:
            acc = acc * float(alpha[e])
        if bias is not None:
            # the reference models round the product to bfloat16 and add the bias in bfloat16
            row = bias[e].cpu().reshape(1, n)
            if out_dtype == torch.bfloat16:
                acc = (acc.to(torch.bfloat16) + row.to(torch.bfloat16)).float()
            else:
                acc = acc + row.float()
        out[rows] = acc
    return out.to(out_dtype)
