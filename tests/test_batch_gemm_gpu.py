"""GPU parity tests of ``batch_gemm`` against the CPU per-batch dequantise-then-matmul
oracle.  Mirrors the reference's ``tests/test_batch_gemm.py`` (its shape lists,
tiles that straddle two batches, per-batch bias and alpha, error texts,
determinism).  Calls go through the Python wrapper and therefore the C ABI.

Tolerances as for ``dense_gemm``: ``rtol 2e-2 / atol 2e-3`` (MXFP8; with a bias the
reference's ``atol`` grows to 1e-2 since it rounds to bfloat16 before adding) and
``5e-2 / 5e-2`` (FP4)."""

import re

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

W8A8_TOL = dict(rtol=2e-2, atol=2e-3)
W4A4_TOL = dict(rtol=5e-2, atol=5e-2)


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _inputs(hq, b, m, n, k, mode, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn([b, m, k], generator=g).to(torch.bfloat16).cuda()
    w = torch.randn([b, n, k], generator=g).to(torch.bfloat16).cuda()
    xq, sfa = hq.group_wise_quant(x.view(b * m, k), mode=mode)
    if n % 128 == 0:
        wq, sfb = hq.group_wise_quant(w.view(b * n, k), mode=mode)
        return xq.view(b, m, -1), wq.view(b, n, -1), sfa, sfb.view(b, n, -1)
    # each batch's weight scales start on their own 128-row atom
    parts = [hq.group_wise_quant(w[i], mode=mode) for i in range(b)]
    wq = torch.stack([p[0] for p in parts])
    sfb = torch.stack([p[1] for p in parts])
    return xq.view(b, m, -1), wq, sfa, sfb


def _run(hq, xq, wq, sfa, sfb, mode, bias=None, alpha=None, **kw):
    b, m, n = xq.shape[0], xq.shape[1], wq.shape[1]
    out = torch.full([m, b * n], float("nan"), dtype=torch.bfloat16, device="cuda")
    hq.batch_gemm(xq, wq, sfa, sfb, out, bias, alpha, mode=mode, **kw)
    assert hq.device_status() == 0
    return out


def _compare(out, xq, wq, sfa, sfb, mode, bias=None, alpha=None):
    ref = oracle.batch_gemm_ref(xq, wq, sfa, sfb, mode, alpha=None if alpha is None else alpha.cpu(),
                                bias=bias)
    tol = dict(W8A8_TOL if mode == "w8a8-mxfp8" else W4A4_TOL)
    if bias is not None:
        tol["atol"] = 1e-2
    torch.testing.assert_close(out.float().cpu(), ref.float(), **tol)


@pytest.mark.parametrize("b,m,n,k,add_bias", [
    (4, 128, 256, 128, False), (4, 1024, 256, 128, False), (2, 256, 128, 128, True), (1, 64, 128, 256, False),
    (1, 256, 256, 128, False), (2, 128, 256, 512, False), (8, 1, 1024, 256, False), (3, 100, 256, 256, False),
    (3, 200, 256, 128, False), (8, 1000, 1024, 256, False), (2, 640, 256, 128, False),
    (2, 2176, 256, 128, False), (2, 640, 128, 128, True), (2, 1000, 256, 128, False), (3, 300, 128, 128, True),
    (2, 5, 256, 256, False), (5, 77, 192, 384, True), (16, 130, 512, 1024, False)], ids=lambda v: str(v))
def test_mxfp8(hq, b, m, n, k, add_bias):
    """Reference shape list (tests/test_batch_gemm.py:237-262) plus a 64-wide-tile and a
    many-straddles case."""
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w8a8-mxfp8")
    bias = None
    if add_bias:
        bias = torch.rand([b, n], generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).cuda()
    out = _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8", bias=bias)
    _compare(out, xq, wq, sfa, sfb, "w8a8-mxfp8", bias=bias)


@pytest.mark.parametrize("mode,k", [("w4a4-nvfp4", 256), ("w4a4-mxfp4", 512)])
@pytest.mark.parametrize("b,m,n", [(4, 128, 256), (4, 1024, 256), (1, 64, 128), (1, 256, 256), (3, 200, 256)],
                         ids=lambda v: str(v))
def test_fp4(hq, mode, k, b, m, n):
    """tests/test_batch_gemm.py:485-497,611-619 (K doubled for the 64-row case there)."""
    if m == 64:
        k = 512
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, mode)
    alpha = None
    if mode == "w4a4-nvfp4":
        alpha = (0.5 + torch.arange(b, dtype=torch.float32) * 0.25).cuda()
    out = _run(hq, xq, wq, sfa, sfb, mode, alpha=alpha)
    _compare(out, xq, wq, sfa, sfb, mode, alpha=alpha)


@pytest.mark.parametrize("tile", ["pair256", "pair128"])
@pytest.mark.parametrize("b,m,n,k,add_bias", [(3, 512, 512, 256, True), (2, 256, 256, 128, False),
                                              (4, 1024, 256, 384, False)], ids=lambda v: str(v))
def test_2cta_tile(hq, monkeypatch, tile, b, m, n, k, add_bias):
    """Batches of a multiple of 256 rows run on the 2-CTA tile, with the same bits as the single-CTA tiles."""
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w8a8-mxfp8", seed=5)
    bias = None
    if add_bias:
        bias = torch.rand([b, n], generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).cuda()
    monkeypatch.setenv("HALOPS_B200_TILE", tile)
    assert "pair=1" in hq.describe_group_tile("batch", b, m, n, k)
    out = _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8", bias=bias)
    _compare(out, xq, wq, sfa, sfb, "w8a8-mxfp8", bias=bias)
    monkeypatch.setenv("HALOPS_B200_TILE", "128")
    assert torch.equal(out, _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8", bias=bias))


@pytest.mark.parametrize("tile", ["256", "128", "64"])
def test_every_tile_width(hq, monkeypatch, tile):
    """Each single-CTA tile width walks the batches the same way."""
    monkeypatch.setenv("HALOPS_B200_TILE", tile)
    xq, wq, sfa, sfb = _inputs(hq, 3, 200, 512, 256, "w8a8-mxfp8", seed=3)
    out = _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8")
    _compare(out, xq, wq, sfa, sfb, "w8a8-mxfp8")


def test_matches_dense_per_batch(hq):
    """Bit-exact against dense_gemm on each batch (same kernel, same tile, same k order)."""
    b, m, n, k = 3, 256, 512, 512
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w8a8-mxfp8", seed=5)
    out = _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8")
    sfa_b = sfa.view(b, m, -1)  # M % 128 == 0: each batch owns whole atoms
    for i in range(b):
        d = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
        hq.dense_gemm(xq[i], wq[i], sfa_b[i].contiguous(), sfb[i].contiguous(), d)
        assert torch.equal(d, out[:, i * n:(i + 1) * n])


def test_strided_output_and_untouched_columns(hq):
    b, m, n, k = 2, 100, 128, 128
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w8a8-mxfp8", seed=6)
    wide = torch.full([m, b * n + 64], 7.0, dtype=torch.bfloat16, device="cuda")
    out = wide[:, : b * n]
    hq.batch_gemm(xq, wq, sfa, sfb, out)
    assert hq.device_status() == 0
    _compare(out, xq, wq, sfa, sfb, "w8a8-mxfp8")
    assert torch.all(wide[:, b * n:] == 7.0)


def test_determinism_pdl_sm_count(hq):
    xq, wq, sfa, sfb = _inputs(hq, 4, 300, 256, 256, "w8a8-mxfp8", seed=7)
    first = _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8", use_pdl=False)
    for kw in (dict(use_pdl=True), dict(sm_count=7), dict(sm_count=148)):
        assert torch.equal(first, _run(hq, xq, wq, sfa, sfb, "w8a8-mxfp8", **kw))


def _empty(b=2, m=128, n=256, k=128, x_shape=None, w_shape=None, out_shape=None):
    x = torch.empty(x_shape or [b, m, k], dtype=torch.float8_e4m3fn, device="cuda")
    w = torch.empty(w_shape or [b, n, k], dtype=torch.float8_e4m3fn, device="cuda")
    sfa = torch.empty([b * m, k // 32], dtype=torch.uint8, device="cuda")
    sfb = torch.empty([b, n, k // 32], dtype=torch.uint8, device="cuda")
    out = torch.empty(out_shape or [m, b * n], dtype=torch.bfloat16, device="cuda")
    return x, w, sfa, sfb, out


@pytest.mark.parametrize("k,x_shape,w_shape,out_shape,mode,expected", [
    (128, None, None, None, "w2a2", "Unsupported mode"),
    (128, [256, 128], None, None, "w8a8-mxfp8", "input must be a 3D tensor"),
    (128, None, [3, 256, 128], None, "w8a8-mxfp8", "weight batch dim must match"),
    (128, None, None, [2, 128, 256], "w8a8-mxfp8", "output must be a 2D tensor"),
    (96, None, None, None, "w8a8-mxfp8", "No batch w8a8-mxfp8 tile for M=128 (grid M=256), N=256, K=96"),
], ids=["bad_mode", "bad_input_rank", "bad_weight_batch", "bad_output_rank", "bad_k"])
def test_mxfp8_errors(hq, k, x_shape, w_shape, out_shape, mode, expected):
    """tests/test_batch_gemm.py:313-363."""
    x, w, sfa, sfb, out = _empty(k=k, x_shape=x_shape, w_shape=w_shape, out_shape=out_shape)
    with pytest.raises(RuntimeError, match=re.escape(expected)):
        hq.batch_gemm(x, w, sfa, sfb, out, None, None, -1, mode)


def test_fp4_errors(hq):
    """tests/test_batch_gemm.py:537-590,658-700."""
    b, m, n, k = 2, 128, 256, 256
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w4a4-nvfp4")
    out = torch.empty([m, b * n], dtype=torch.bfloat16, device="cuda")
    alpha = torch.ones([b], dtype=torch.float32, device="cuda")
    bias = torch.zeros([b, n], dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="requires alpha input"):
        hq.batch_gemm(xq, wq, sfa, sfb, out, None, None, -1, "w4a4-nvfp4")
    with pytest.raises(RuntimeError, match="W4A4 batch GEMM does not support bias"):
        hq.batch_gemm(xq, wq, sfa, sfb, out, bias, alpha, -1, "w4a4-nvfp4")
    with pytest.raises(RuntimeError, match="packed input K/2 must match packed weight K/2"):
        hq.batch_gemm(xq, wq[:, :, :64].contiguous(), sfa, sfb, out, None, alpha, -1, "w4a4-nvfp4")
    with pytest.raises(RuntimeError, match="W4A4 scale-factor shape does not match mode"):
        hq.batch_gemm(xq, wq, sfa, sfb, out, None, None, -1, "w4a4-mxfp4")
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, 512, "w4a4-mxfp4")
    with pytest.raises(RuntimeError, match="does not take alpha"):
        hq.batch_gemm(xq, wq, sfa, sfb, out, None, alpha, -1, "w4a4-mxfp4")
    with pytest.raises(RuntimeError, match="W4A4 batch GEMM does not support bias"):
        hq.batch_gemm(xq, wq, sfa, sfb, out, bias, None, -1, "w4a4-mxfp4")


def test_other_epilogues_raise(hq):
    x, w, sfa, sfb, out = _empty()
    with pytest.raises(RuntimeError, match="Unsupported epilogue 3"):
        hq.batch_gemm(x, w, sfa, sfb, out, epilogue=hq.EpilogueOp.Sigmoid)
    with pytest.raises(RuntimeError, match="GateMulQuant epilogues need gate"):
        hq.batch_gemm(x, w, sfa, sfb, out, epilogue=hq.EpilogueOp.GateMulQuant)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4"])
def test_golden_fixture(hq, golden_dir, mode):
    """Inputs and outputs of the reference's own input builders and CPU model
    (tests/golden/make_golden.py); the MXFP8 case has 100 rows per batch and a bias."""
    import os

    import numpy as np

    def bf16(bits):
        return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)

    d = np.load(os.path.join(golden_dir, f"batch_{mode}.npz"))
    x, w = torch.from_numpy(d["x"]).cuda(), torch.from_numpy(d["w"]).cuda()
    if mode == "w8a8-mxfp8":
        x, w = x.view(torch.float8_e4m3fn), w.view(torch.float8_e4m3fn)
    sfa, sfb = torch.from_numpy(d["sfa"]).cuda(), torch.from_numpy(d["sfb"]).cuda()
    alpha = torch.from_numpy(d["alpha"]).cuda() if "alpha" in d else None
    bias = bf16(d["bias_bits"]).cuda() if "bias_bits" in d else None
    out = _run(hq, x, w, sfa, sfb, mode, bias=bias, alpha=alpha)
    ref = bf16(d["out_bits"]).float()  # [B, M, N]
    tol = dict(W8A8_TOL if mode == "w8a8-mxfp8" else W4A4_TOL)
    if bias is not None:
        tol["atol"] = 1e-2
    n = w.shape[1]
    for b in range(x.shape[0]):
        torch.testing.assert_close(out[:, b * n:(b + 1) * n].float().cpu(), ref[b], **tol)


def _ref_quant_e4m3(v):
    """Per-32-column MXFP8 model of the quantising epilogues: e4m3 codes and UE8M0 exponents
    (the reference's ``ref_quant_e4m3``, tests/test_batch_gemm.py:389-396)."""
    g = v.float().unflatten(-1, (-1, 32))
    amax = g.abs().amax(-1).clamp_min(1e-10)
    mant, exp = torch.frexp(amax)
    e = (exp - 9 + (mant > 0.875).int() + 127).clamp(0, 254)
    q = (g * torch.exp2(127 - e.float())[..., None]).flatten(-2)
    return q.to(torch.float8_e4m3fn).view(torch.uint8), e.to(torch.uint8)


def _quant_run(hq, args, m, cols, op, gate):
    out = torch.empty([m, cols], dtype=torch.float8_e4m3fn, device="cuda")
    # not cleared by the caller: the kernel writes the zero bytes of the padding rows itself
    out_sf = torch.full([(m + 127) // 128 * 128 * cols // 32], 0xAB, dtype=torch.uint8, device="cuda")
    hq.batch_gemm(*args, out, None, None, -1, "w8a8-mxfp8", op, out_sf, gate)
    assert hq.device_status() == 0
    return out.view(torch.uint8), out_sf


@pytest.mark.parametrize("with_gate", [False, True], ids=["quant", "gate_mul"])
@pytest.mark.parametrize("b,m,n,k", [(3, 200, 256, 128), (8, 200, 1024, 2048), (2, 128, 128, 256)],
                         ids=lambda v: str(v))
def test_e4m3_out(hq, b, m, n, k, with_gate):
    """The e4m3 output and its scales equal the bf16 output (times gate) quantised per 32
    columns, bit for bit; the scale bytes of the padding rows are zero (tests/test_batch_gemm.py:399-434
    there, which clears the buffer first; here the kernel does it)."""
    import numpy as np

    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w8a8-mxfp8", seed=11)
    args = (xq, wq, sfa, sfb)
    y = _run(hq, *args, "w8a8-mxfp8")
    gate = None
    if with_gate:
        gate = (torch.rand([m, b * n], generator=torch.Generator().manual_seed(12)) * 2 - 0.5).to(torch.bfloat16).cuda()
    ref_q, ref_sf = _ref_quant_e4m3((y * gate if with_gate else y).cpu())
    op = hq.EpilogueOp.GateMulQuant if with_gate else hq.EpilogueOp.Quant
    q, sf = _quant_run(hq, args, m, b * n, op, gate)
    assert torch.equal(q.cpu(), ref_q)
    idx = torch.from_numpy(oracle.sf_atom_offsets(m, b * n // 32))
    assert torch.equal(sf.cpu()[idx], ref_sf)
    pad = torch.ones(sf.numel(), dtype=torch.bool)
    pad[idx.flatten()] = False
    assert (sf.cpu()[pad] == 0).all()
    q2, sf2 = _quant_run(hq, args, m, b * n, op, gate)
    assert torch.equal(q, q2) and torch.equal(sf, sf2)
    del np


@pytest.mark.parametrize("b,m,n,k", [(3, 200, 256, 128), (8, 200, 1024, 2048)], ids=lambda v: str(v))
def test_sigmoid_gate_mul_quant(hq, b, m, n, k):
    """A gate read in place from a column slice of a wider tensor equals its contiguous copy;
    SigmoidGateMulQuant on logits matches GateMulQuant on bf16(sigmoid(logits)) up to the
    sigmoid's rounding: codes within 1 where the scale matches, at most 0.1 % of the scales
    off by one (tests/test_batch_gemm.py:447-482)."""
    xq, wq, sfa, sfb = _inputs(hq, b, m, n, k, "w8a8-mxfp8", seed=13)
    args = (xq, wq, sfa, sfb)
    cols = b * n
    wide = (torch.randn([m, 3 * cols], generator=torch.Generator().manual_seed(14)) * 3).to(torch.bfloat16).cuda()
    logits = wide[:, cols:2 * cols]
    q, sf = _quant_run(hq, args, m, cols, hq.EpilogueOp.GateMulQuant, logits)
    ref_q, ref_sf = _quant_run(hq, args, m, cols, hq.EpilogueOp.GateMulQuant, logits.contiguous())
    assert torch.equal(q, ref_q) and torch.equal(sf, ref_sf)

    q, sf = _quant_run(hq, args, m, cols, hq.EpilogueOp.SigmoidGateMulQuant, logits)
    gate = torch.sigmoid(logits.float()).to(torch.bfloat16)
    ref_q, ref_sf = _quant_run(hq, args, m, cols, hq.EpilogueOp.GateMulQuant, gate)
    sf_diff = (sf.int() - ref_sf.int()).abs().cpu()
    assert sf_diff.max() <= 1 and (sf_diff > 0).float().mean() <= 1e-3
    idx = torch.from_numpy(oracle.sf_atom_offsets(m, cols // 32))
    same_scale = (sf_diff[idx] == 0).repeat_interleave(32, -1)

    def ordered(t):
        i = t.cpu().view(torch.int8).to(torch.int32)
        return torch.where(i < 0, -(i & 127), i)

    code_diff = (ordered(q) - ordered(ref_q)).abs()
    assert code_diff[same_scale].max() <= 1


def test_quant_epilogue_rules(hq):
    x, w, sfa, sfb, out = _empty()
    q = torch.empty([128, 512], dtype=torch.float8_e4m3fn, device="cuda")
    sf = torch.zeros([128 * 16], dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        hq.batch_gemm(x, w, sfa, sfb, out, epilogue=hq.EpilogueOp.Quant, output_sf=sf)
    with pytest.raises(RuntimeError, match="need a contiguous uint8 output_sf"):
        hq.batch_gemm(x, w, sfa, sfb, q, epilogue=hq.EpilogueOp.Quant)
    with pytest.raises(RuntimeError, match="output_sf must hold whole 128-row SfAtoms"):
        hq.batch_gemm(x, w, sfa, sfb, q, epilogue=hq.EpilogueOp.Quant, output_sf=sf[:100])
    gate = torch.zeros([128, 512 + 8], dtype=torch.bfloat16, device="cuda")[:, 8:]
    with pytest.raises(RuntimeError, match="32-byte aligned"):
        hq.batch_gemm(x, w, sfa, sfb, q, epilogue=hq.EpilogueOp.GateMulQuant, output_sf=sf, gate=gate)
    xq, wq, sfa4, sfb4 = _inputs(hq, 2, 128, 256, 256, "w4a4-nvfp4")
    alpha = torch.ones([2], dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="Unsupported epilogue 1 for w4a4-nvfp4"):
        hq.batch_gemm(xq, wq, sfa4, sfb4, q, None, alpha, -1, "w4a4-nvfp4", hq.EpilogueOp.Quant, sf)
