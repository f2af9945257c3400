"""Multi-threaded CPU path of the reference for timing: MXFP8 quantise +
dequantise + float32 matmul with torch ops on all host cores.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``); used by the benchmark's
CPU-baseline legs, never by the library.

Follows the reference's torch helpers: ``per_token_cast_to_fp8``
(``tests/utils/gemm_utils.py:88-108``) for the quantiser and ``ref_gemm``
(``tests/test_dense_gemm.py:48-65``) for the GEMM.  The scale exponent uses
the bit-field form of ``oracle.quant.ue8m0_from_scale_closed_form`` so that
the bytes equal the numpy oracle's (checked in ``tests/test_oracle_golden.py``).
"""

from __future__ import annotations

import torch


def quant_mxfp8_torch(x: torch.Tensor):
    """[m, k] bf16 -> ([m, k] float8_e4m3fn, [m, k/32] uint8 logical UE8M0 scales)."""
    m, k = x.shape
    xg = x.reshape(m, k // 32, 32).to(torch.float32)
    amax = xg.abs().amax(dim=-1).clamp(min=1e-10)
    scale = amax / 448.0
    raw = scale.view(torch.int32)
    exp = (raw >> 23) & 0xFF
    man = raw & 0x007FFFFF
    e = (exp + ((man != 0) | (exp < 127)).to(torch.int32)).clamp(0, 254)
    inv = ((254 - e) << 23).view(torch.float32)
    q = (xg * inv.unsqueeze(-1)).clamp(-448.0, 448.0).reshape(m, k).to(torch.float8_e4m3fn)
    return q, e.to(torch.uint8)


def dequant_mxfp8_torch(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    scale = torch.exp2(sf.to(torch.float32) - 127.0)
    return q.to(torch.float32) * torch.repeat_interleave(scale, 32, dim=1)


def gemm_mxfp8_torch(aq, sfa, bq, sfb) -> torch.Tensor:
    """bf16(dequant(A) @ dequant(B)^T) in float32 on the CPU."""
    return torch.matmul(dequant_mxfp8_torch(aq, sfa), dequant_mxfp8_torch(bq, sfb).T).to(torch.bfloat16)
