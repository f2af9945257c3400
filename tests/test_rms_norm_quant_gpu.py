"""GPU parity tests of ``rms_norm_quant`` (mirrors the reference's
``tests/test_rms_norm_quant.py``).  The fused kernel's bf16 norm may differ
from the oracle's fp32 RMSNorm by one bf16 ulp (summation order, rsqrt), which
moves a code by at most one step or, rarely, a group's amax across a power of
two: codes match within 1 where the scale matches and at most 0.1 % of the
scales differ, each by 1 - the reference's own tolerance."""

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
EPS = 1e-6


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _inputs(m, k, seed=0):
    g = torch.Generator().manual_seed(seed + m * 7 + k)
    x = (torch.randn([m, k], generator=g) * 3).to(torch.bfloat16)
    w = (torch.rand([k], generator=g) + 0.5).to(torch.bfloat16)
    return x, w


def _ulp_diff(a, b):
    def ordered(t):
        i = t.astype(np.int8).astype(np.int32)
        return np.where(i < 0, -(i & 0x7F), i)

    return np.abs(ordered(a) - ordered(b))


@pytest.mark.parametrize("use_swizzle", [True, False], ids=["sfatom", "rowmajor"])
@pytest.mark.parametrize("k", [128, 1024, 4096, 8192])
@pytest.mark.parametrize("m", [1, 16, 128, 200, 1536, 3072])
def test_rms_norm_quant(hq, m, k, use_swizzle):
    x, w = _inputs(m, k)
    q, sf = hq.rms_norm_quant(x.cuda(), w.cuda(), EPS, use_swizzle=use_swizzle)
    assert q.dtype == torch.float8_e4m3fn and list(q.shape) == [m, k]
    assert list(sf.shape) == [(m + 127) // 128 * 128 if use_swizzle else m, k // 32]
    ref_q, ref_sf = oracle.quant_group_wise(oracle.rms_norm_ref(x, w, EPS), "w8a8-mxfp8", use_swizzle)
    q, sf = q.view(torch.uint8).cpu().numpy(), sf.cpu().numpy()
    if use_swizzle:
        full = oracle.unswizzle_sf(sf, sf.shape[0])
        assert not full[m:].any(), "padding rows of the last scale atom must be zero"
        sf, ref_sf = full[:m], oracle.unswizzle_sf(ref_sf, m)
    sf_diff = np.abs(sf.astype(np.int32) - ref_sf.astype(np.int32))
    assert sf_diff.max() <= 1 and (sf_diff > 0).mean() <= 1e-3
    same = np.repeat(sf_diff == 0, 32, axis=1)
    assert _ulp_diff(q, ref_q)[same].max() <= 1
    assert (q != ref_q)[same].mean() < 0.02


def test_matches_unfused_pipeline_closely(hq):
    """Against this library's own group_wise_quant of a torch bf16 RMSNorm on the GPU."""
    x, w = _inputs(512, 4096, 3)
    xg, wg = x.cuda(), w.cuda()
    q, sf = hq.rms_norm_quant(xg, wg, EPS)
    y = (xg.float() * torch.rsqrt(xg.float().pow(2).mean(-1, keepdim=True) + EPS) * wg.float()).to(torch.bfloat16)
    rq, rsf = hq.group_wise_quant(y)
    assert (sf != rsf).float().mean() <= 1e-3
    assert (q.view(torch.uint8) != rq.view(torch.uint8)).float().mean() < 0.02


@pytest.mark.parametrize("m", [1, 200])
def test_strided_input_pdl_and_determinism(hq, m):
    k = 1024
    x, w = _inputs(m, 2 * k, 5)
    xs, ws = x.cuda()[:, k:], w.cuda()[:k].contiguous()
    ref_q, ref_sf = hq.rms_norm_quant(xs.contiguous(), ws, EPS, use_pdl=False)
    for _ in range(3):
        q, sf = hq.rms_norm_quant(xs, ws, EPS)
        assert torch.equal(q.view(torch.uint8), ref_q.view(torch.uint8)) and torch.equal(sf, ref_sf)


def test_empty_and_errors(hq):
    x, w = _inputs(0, 1024)
    q, sf = hq.rms_norm_quant(x.cuda(), w.cuda(), EPS)
    assert q.shape == (0, 1024) and sf.shape == (0, 32)
    x, w = _inputs(4, 1056)
    with pytest.raises(RuntimeError, match="K must be a multiple of 128"):
        hq.rms_norm_quant(x.cuda(), w.cuda())
    x, w = _inputs(4, 1024)
    with pytest.raises(RuntimeError, match="weight must be a contiguous bfloat16"):
        hq.rms_norm_quant(x.cuda(), w.cuda()[:512])
    with pytest.raises(RuntimeError, match="2D bfloat16"):
        hq.rms_norm_quant(x.cuda().float(), w.cuda())


def test_feeds_dense_gemm(hq):
    """rms_norm_quant -> dense_gemm equals group_wise_quant(norm) -> dense_gemm up to the 1-ulp norm differences."""
    m, n, k = 256, 512, 2048
    x, w = _inputs(m, k, 9)
    g = torch.Generator().manual_seed(1)
    wt = (torch.randn([n, k], generator=g) * 0.05).to(torch.bfloat16).cuda()
    bq, sfb = hq.group_wise_quant(wt)
    aq, sfa = hq.rms_norm_quant(x.cuda(), w.cuda(), EPS)
    out = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, out)
    ref = oracle.rms_norm_ref(x, w, EPS).float() @ wt.float().cpu().T
    rel = (out.float().cpu() - ref).norm() / ref.norm()
    assert rel < 0.05


def test_golden_fixture(hq, golden_dir):
    """Inputs of the reference's own builder and its fp32 RMSNorm rounded to bf16
    (tests/golden/make_golden.py), quantised by the pinned oracle: same bound as above."""
    import os

    d = np.load(os.path.join(golden_dir, "rms_norm.npz"))
    bf16 = lambda bits: torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)  # noqa: E731
    x, w, y = bf16(d["x_bits"]), bf16(d["w_bits"]), bf16(d["y_bits"])
    q, sf = hq.rms_norm_quant(x.cuda(), w.cuda(), float(d["eps"]), use_swizzle=False)
    ref_q, ref_sf = oracle.quant_group_wise(y, "w8a8-mxfp8", False)
    q, sf = q.view(torch.uint8).cpu().numpy(), sf.cpu().numpy()
    sf_diff = np.abs(sf.astype(np.int32) - ref_sf.astype(np.int32))
    assert sf_diff.max() <= 1 and (sf_diff > 0).mean() <= 1e-3
    same = np.repeat(sf_diff == 0, 32, axis=1)
    assert _ulp_diff(q, ref_q)[same].max() <= 1
