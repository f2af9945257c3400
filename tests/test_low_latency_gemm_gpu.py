"""GPU parity tests of ``low_latency_mma_gemm`` (M <= 16, plain row-major scales) against
the CPU dequantise-then-matmul oracle.  Mirrors the reference's
``tests/test_low_latency_mma_gemm.py``: its shape list (N a multiple of 8 only, K blocks
not a power of two, padded and strided scale rows, very large K), dual output, concat-K,
sigmoid, grid-size independence and the rejects.  Inputs scale every (row, 32-wide K group)
by its own power of two, so a scale read from the wrong row or group shows up as a factor
of two.  Tolerance: the reference's ``rtol 2e-2 / atol 2e-3``."""

import re

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = dict(rtol=2e-2, atol=2e-3)


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _spread_groups(values, g):
    rows, cols = values.shape
    exponents = torch.randint(-2, 3, (rows, cols // 32, 1), generator=g).float()
    return (values.float().view(rows, cols // 32, 32) * torch.exp2(exponents)).view(rows, cols).to(torch.bfloat16)


def _make_bf16(rows, cols, magnitude, g):
    return _spread_groups(torch.randn(rows, cols, generator=g).to(torch.bfloat16) * magnitude, g)


def _pad_scale_rows(scale, extra_bytes=0):
    rows, cols = scale.shape
    pitch = -(-cols // 16) * 16
    buffer = torch.zeros(rows, pitch + extra_bytes, dtype=torch.uint8, device=scale.device)
    buffer[:, :cols].copy_(scale)
    return buffer[:, :cols]


def _quant(hq, values):
    q, scale = hq.group_wise_quant(values.cuda(), mode="w8a8-mxfp8", use_swizzle=False)
    if scale.stride(0) % 16:
        scale = _pad_scale_rows(scale)
    return q, scale


def _operands(hq, m, n, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    xq, sfa = _quant(hq, _make_bf16(m, k, 0.1, g))
    wq, sfb = _quant(hq, _make_bf16(n, k, k ** -0.5, g))
    return xq, sfa, wq, sfb


def _reference(xq, sfa, wq, sfb):
    a = oracle.dequantize(xq, sfa.contiguous(), "w8a8-mxfp8", swizzled=False)
    b = oracle.dequantize(wq, sfb.contiguous(), "w8a8-mxfp8", swizzled=False)
    return a @ b.T


def _run(hq, xq, wq, sfa, sfb, **kw):
    out = torch.full([xq.shape[0], wq.shape[0]], float("nan"), dtype=torch.bfloat16, device="cuda")
    hq.low_latency_mma_gemm(xq, wq, sfa, sfb, out, **kw)
    assert hq.device_status() == 0
    return out


def _check(out, expected):
    torch.testing.assert_close(out.float().cpu(), expected, **TOL)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (5, 520, 7168), (8, 2048, 1280), (16, 7168, 2048),
                                   (1, 512, 23808), (16, 8, 256), (3, 72, 512), (16, 512, 16384)],
                         ids=lambda v: str(v))
def test_gemm(hq, m, n, k):
    """tests/test_low_latency_mma_gemm.py:89-101 plus the smallest shape, a two-tile N with a
    tail of 8 and a K the reference rejects for its resident A."""
    xq, sfa, wq, sfb = _operands(hq, m, n, k)
    _check(_run(hq, xq, wq, sfa, sfb), _reference(xq, sfa, wq, sfb))


def test_strided_scales_match_contiguous(hq):
    xq, sfa, wq, sfb = _operands(hq, 8, 512, 4096, seed=1)
    strided = _run(hq, xq, wq, _pad_scale_rows(sfa, 16), _pad_scale_rows(sfb, 16))
    assert torch.equal(strided, _run(hq, xq, wq, sfa, sfb))


def test_sm_count_and_pdl_do_not_change_the_result(hq):
    xq, sfa, wq, sfb = _operands(hq, 8, 4096, 1024, seed=2)
    full = _run(hq, xq, wq, sfa, sfb)
    for kw in (dict(sm_count=1), dict(sm_count=7), dict(use_pdl=False)):
        assert torch.equal(full, _run(hq, xq, wq, sfa, sfb, **kw))


@pytest.mark.parametrize("use_pdl", [True, False])
@pytest.mark.parametrize("m,n,n2,k", [(8, 4096, 1024, 2048), (16, 1544, 520, 1024)], ids=lambda v: str(v))
def test_dual_output(hq, m, n, n2, k, use_pdl):
    xq, sfa, wq, sfb = _operands(hq, m, n, k, seed=3)
    w2q, sfb2 = _quant(hq, _make_bf16(n2, k, k ** -0.5, torch.Generator().manual_seed(4)))
    out2 = torch.full([m, n2], float("nan"), dtype=torch.bfloat16, device="cuda")
    out = _run(hq, xq, wq, sfa, sfb, weight2=w2q, sfb2=sfb2, output2=out2, use_pdl=use_pdl)
    _check(out, _reference(xq, sfa, wq, sfb))
    _check(out2, _reference(xq, sfa, w2q, sfb2))


@pytest.mark.parametrize("use_pdl", [True, False])
@pytest.mark.parametrize("m,n,k1,k2,scale_pad", [(8, 4096, 2048, 2048, 0), (16, 2048, 1024, 768, 16)],
                         ids=lambda v: str(v))
def test_concat_k(hq, m, n, k1, k2, scale_pad, use_pdl):
    xq, sfa, wq, sfb = _operands(hq, m, n, k1, seed=5)
    g = torch.Generator().manual_seed(6)
    x2q, sfa2 = _quant(hq, _make_bf16(m, k2, 0.1, g))
    w2q, sfb2 = _quant(hq, _make_bf16(n, k2, k2 ** -0.5, g))
    if scale_pad:
        sfa, sfb, sfa2, sfb2 = (_pad_scale_rows(s, scale_pad) for s in (sfa, sfb, sfa2, sfb2))
    out = _run(hq, xq, wq, sfa, sfb, input2=x2q, weight2=w2q, sfa2=sfa2, sfb2=sfb2, use_pdl=use_pdl)
    _check(out, _reference(xq, sfa, wq, sfb) + _reference(x2q, sfa2, w2q, sfb2))


@pytest.mark.parametrize("m", [6, 16])
def test_sigmoid(hq, m):
    xq, sfa, wq, sfb = _operands(hq, m, 2048, 1024, seed=7)
    out = _run(hq, xq, wq, sfa, sfb, use_sigmoid=True)
    assert torch.equal(out, torch.sigmoid(_run(hq, xq, wq, sfa, sfb)))


def test_rejects(hq):
    """tests/test_low_latency_mma_gemm.py:226-345."""
    def args(xq, sfa, wq, sfb, **kw):
        out = torch.empty(xq.shape[0], wq.shape[0], dtype=torch.bfloat16, device="cuda")
        return dict(input=xq, weight=wq, sfa=sfa, sfb=sfb, output=out, **kw)

    def raises(text, kw):
        with pytest.raises(RuntimeError, match=re.escape(text)):
            hq.low_latency_mma_gemm(**kw)

    raises("supports M <= 16", args(*_operands(hq, 17, 512, 4096)))
    raises("weight rows must be divisible by 8", args(*_operands(hq, 8, 516, 256)))
    raises("K must be divisible by 256", args(*_operands(hq, 8, 512, 1152)))
    xq, sfa, wq, sfb = _operands(hq, 8, 512, 1024)
    raises("plain row-major", args(xq, _pad_scale_rows(sfa, 4), wq, sfb))
    xq, _, wq, sfb = _operands(hq, 8, 4096, 4096)
    _, swizzled = hq.group_wise_quant(torch.zeros([8, 4096], dtype=torch.bfloat16, device="cuda"), use_swizzle=True)
    raises("plain row-major", args(xq, swizzled, wq, sfb))
    xq, sfa, wq, sfb = _operands(hq, 8, 512, 2048)
    shifted = torch.empty(wq.numel() + 1, dtype=torch.float8_e4m3fn, device="cuda")[1:].view(wq.shape)
    shifted.copy_(wq)
    raises("TMA descriptor encoding failed", args(xq, sfa, shifted, sfb))
    raises("weight2 / sfb2 must come with", args(xq, sfa, wq, sfb, weight2=wq, sfb2=sfb))
    out2 = torch.empty(8, 512, dtype=torch.bfloat16, device="cuda")
    raises("does not support", args(xq, sfa, wq, sfb, weight2=wq, sfb2=sfb, output2=out2, use_sigmoid=True))
    xq, sfa, wq, sfb = _operands(hq, 8, 512, 1920)
    x2q, sfa2, w2q, sfb2 = _operands(hq, 8, 512, 2176)
    raises("K1 must be a multiple of 512", args(xq, sfa, wq, sfb, input2=x2q, weight2=w2q, sfa2=sfa2, sfb2=sfb2))


def test_golden_fixture(hq, golden_dir):
    """Operands built by the reference's own recipe (a power of two per row and k-group,
    its CPU quantizer, plain scales) and the output of its dequantise-then-matmul model
    (tests/golden/make_golden.py); N = 136 is 8-aligned but no multiple of the tile."""
    import os

    import numpy as np

    d = np.load(os.path.join(golden_dir, "low_latency_w8a8-mxfp8.npz"))
    xq = torch.from_numpy(d["x"]).cuda().view(torch.float8_e4m3fn)
    wq = torch.from_numpy(d["w"]).cuda().view(torch.float8_e4m3fn)
    sfa, sfb = _pad_scale_rows(torch.from_numpy(d["sfa"]).cuda()), _pad_scale_rows(torch.from_numpy(d["sfb"]).cuda())
    _check(_run(hq, xq, wq, sfa, sfb), torch.from_numpy(d["out"]))
