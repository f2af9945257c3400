"""GPU parity tests of ``dense_gemm`` against the CPU dequantise-then-matmul
oracle.  Mirrors the reference's ``tests/test_dense_gemm.py`` (shapes, unaligned
M, out-of-bounds sentinels, determinism, PDL, quantize -> GEMM chain) and adds
the benchmark configurations.  Calls go through the Python wrapper and
therefore the C ABI.

Tolerances: the reference's ``rtol 2e-2 / atol 2e-3`` (MXFP8) and ``5e-2 / 5e-2``
(FP4) element-wise, plus max|out - ref| / max|ref| <= 1e-2 against the fp32
oracle."""

import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

W8A8_TOL = dict(rtol=2e-2, atol=2e-3)
W4A4_TOL = dict(rtol=5e-2, atol=5e-2)
MAX_REL = 1e-2


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _rand(m, k, seed, kind="normal"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn([m, k], generator=g)
    if kind == "weight":
        x = x * 0.02
    elif kind == "student_t":
        chi2 = torch.randn([3, m, k], generator=g).pow(2).sum(0)
        x = x / torch.sqrt(chi2 / 3)
    return x.to(torch.bfloat16)


def _quantize(hq, a, b, mode):
    aq, sfa = hq.group_wise_quant(a.cuda(), mode=mode)
    bq, sfb = hq.group_wise_quant(b.cuda(), mode=mode)
    return aq, bq, sfa, sfb


def _gemm(hq, aq, bq, sfa, sfb, mode, alpha=None, use_pdl=False, sm_count=-1):
    out = torch.zeros([aq.shape[0], bq.shape[0]], dtype=torch.bfloat16, device="cuda")
    al = None
    if mode == "w4a4-nvfp4":
        al = torch.full([1], 1.0 if alpha is None else alpha, dtype=torch.float32, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, out, None, al, sm_count, mode, use_pdl)
    assert hq.device_status() == 0
    return out


def _check(out, aq, bq, sfa, sfb, mode, alpha=None, rows=None):
    """Compare with the oracle; ``rows`` restricts the check to a row sample."""
    a_sel = aq if rows is None else aq[rows]
    a_deq = oracle.dequantize(aq, sfa, mode)
    if rows is not None:
        a_deq = a_deq[rows]
    b_deq = oracle.dequantize(bq, sfb, mode)
    ref = a_deq @ b_deq.T
    if alpha is not None:
        ref = ref * alpha
    got = (out if rows is None else out[rows]).float().cpu()
    tol = W8A8_TOL if mode == "w8a8-mxfp8" else W4A4_TOL
    torch.testing.assert_close(got, ref.to(torch.bfloat16).float(), **tol)
    rel = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert rel <= MAX_REL, f"max relative error {rel}"
    del a_sel
    return rel


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (128, 256, 256), (64, 128, 256), (128, 128, 128),
                                   (256, 512, 1024), (64, 7168, 3584), (4096, 7168, 3584)],
                         ids=lambda v: str(v))
def test_mxfp8_shapes(hq, m, n, k):
    """Reference shapes (tests/test_dense_gemm.py:186-212) plus config 1 (128x256x512)."""
    a, b = _rand(m, k, 1), _rand(n, k, 2)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    out = _gemm(hq, aq, bq, sfa, sfb, "w8a8-mxfp8")
    _check(out, aq, bq, sfa, sfb, "w8a8-mxfp8")


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4"])
def test_golden_fixture(hq, golden_dir, mode):
    """Operands quantised by the reference's Python helpers (weights with
    32x32 / 16x16 block scales), output produced by the reference's ref_gemm."""
    d = np.load(os.path.join(golden_dir, f"gemm_{mode}.npz"))
    x = torch.from_numpy(d["x"]).cuda()
    w = torch.from_numpy(d["w"]).cuda()
    if mode == "w8a8-mxfp8":
        x, w = x.view(torch.float8_e4m3fn), w.view(torch.float8_e4m3fn)
    sfa, sfb = torch.from_numpy(d["sfa"]).cuda(), torch.from_numpy(d["sfb"]).cuda()
    out = _gemm(hq, x, w, sfa, sfb, mode)
    ref = torch.from_numpy(d["out_bits"].view(np.int16)).view(torch.bfloat16).float()
    tol = W8A8_TOL if mode == "w8a8-mxfp8" else W4A4_TOL
    torch.testing.assert_close(out.float().cpu(), ref, **tol)


@pytest.mark.parametrize("mode, m, n, k", [
    ("w8a8-mxfp8", 129, 1024, 1024), ("w8a8-mxfp8", 200, 1024, 1024), ("w8a8-mxfp8", 300, 1024, 1024),
    ("w8a8-mxfp8", 449, 1024, 1024), ("w8a8-mxfp8", 200, 8192, 4096), ("w8a8-mxfp8", 1000, 8192, 4096),
    ("w8a8-mxfp8", 1, 1024, 1024), ("w8a8-mxfp8", 17, 192, 384),
    ("w4a4-nvfp4", 129, 1024, 1024), ("w4a4-nvfp4", 200, 1024, 1024), ("w4a4-nvfp4", 300, 1024, 1024),
    ("w4a4-mxfp4", 129, 1024, 1024), ("w4a4-mxfp4", 200, 1024, 1024), ("w4a4-mxfp4", 300, 1024, 1024)],
    ids=lambda v: str(v))
def test_unaligned_m(hq, mode, m, n, k):
    """Neither the activation nor the output is padded to 128 rows."""
    a, b = _rand(m, k, 3), _rand(n, k, 4)
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    out = _gemm(hq, aq, bq, sfa, sfb, mode)
    _check(out, aq, bq, sfa, sfb, mode, alpha=1.0 if mode == "w4a4-nvfp4" else None)


@pytest.mark.parametrize("m", [1, 8, 32, 64, 128])
@pytest.mark.parametrize("n,k", [(7168, 2048), (24576, 1536)])
def test_decode_shapes(hq, m, n, k):
    """Config 3: heavy-tailed Student-t activations, N(0, 0.02) weights."""
    a, b = _rand(m, k, 5, "student_t"), _rand(n, k, 6, "weight")
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    out = _gemm(hq, aq, bq, sfa, sfb, "w8a8-mxfp8")
    _check(out, aq, bq, sfa, sfb, "w8a8-mxfp8")


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (256, 384, 768), (4096, 7168, 3584)], ids=lambda v: str(v))
@pytest.mark.parametrize("mode", ["w4a4-nvfp4", "w4a4-mxfp4"])
def test_fp4_shapes(hq, mode, m, n, k):
    a, b = _rand(m, k, 7), _rand(n, k, 8)
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    out = _gemm(hq, aq, bq, sfa, sfb, mode)
    _check(out, aq, bq, sfa, sfb, mode, alpha=1.0 if mode == "w4a4-nvfp4" else None)


def test_nvfp4_alpha_is_applied(hq):
    a, b = _rand(256, 1024, 9), _rand(512, 1024, 10)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w4a4-nvfp4")
    out = _gemm(hq, aq, bq, sfa, sfb, "w4a4-nvfp4", alpha=0.37)
    _check(out, aq, bq, sfa, sfb, "w4a4-nvfp4", alpha=0.37)


def test_config4_nvfp4_full_size(hq):
    """Config 4: M=4096, N=14336, K=4096, checked on a 256-row sample."""
    m, n, k = 4096, 14336, 4096
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.randn([m, k], generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn([n, k], generator=g, device="cuda").to(torch.bfloat16)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w4a4-nvfp4")
    out = _gemm(hq, aq, bq, sfa, sfb, "w4a4-nvfp4")
    _check(out, aq, bq, sfa, sfb, "w4a4-nvfp4", alpha=1.0, rows=torch.arange(0, m, 16))


def test_config2_large_square_sample_and_linearity(hq):
    """Config 2: M=N=K=8192, A ~ N(0,1), B ~ N(0,0.02).  A 256-row sample is
    checked against the oracle; the whole output is checked through a
    size-independent property: scaling one operand's block scales by 2 (adding 1
    to every UE8M0 byte) doubles the output exactly."""
    m = n = k = 8192
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn([m, k], generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn([n, k], generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    out = _gemm(hq, aq, bq, sfa, sfb, "w8a8-mxfp8")
    _check(out, aq, bq, sfa, sfb, "w8a8-mxfp8", rows=torch.arange(0, m, 32))
    out2 = _gemm(hq, aq, bq, sfa, sfb + 1, "w8a8-mxfp8")
    assert torch.equal(out2.float(), out.float() * 2)


def test_config5_shard_sample_and_linearity(hq):
    """The N-sharded configuration, one rank's share of 8: M=16384, N=7168, K=8192,
    activation ~ N(0,1), weight ~ N(0,0.02), on the tile the dispatch picks for it (the
    2-CTA 256x256 one).  A row sample is checked against the oracle; the whole output
    through the exact-doubling property of the block scales."""
    m, n, k = 16384, 7168, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn([m, k], generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn([n, k], generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    assert "pair=1" in hq.describe_tile(m, n, k, "w8a8-mxfp8")
    out = _gemm(hq, aq, bq, sfa, sfb, "w8a8-mxfp8")
    _check(out, aq, bq, sfa, sfb, "w8a8-mxfp8", rows=torch.arange(0, m, 128) + torch.arange(128) % 128)
    out2 = _gemm(hq, aq, bq, sfa + 1, sfb, "w8a8-mxfp8")
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.parametrize("m,n,k", [(8192, 8192, 8192), (16384, 7168, 8192)], ids=lambda v: str(v))
def test_pair_tile_at_benchmark_sizes_200_runs(hq, monkeypatch, m, n, k):
    """At the sizes the dispatch uses it for, the 2-CTA kernel (two MMA-issuing threads taking
    turns per k-tile) gives the single-CTA tile's bits, 200 runs in a row."""
    g = torch.Generator(device="cuda").manual_seed(6)
    a = torch.randn([m, k], generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn([n, k], generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    monkeypatch.setenv("HALOPS_B200_TILE", "256")
    assert "pair=0" in hq.describe_tile(m, n, k, "w8a8-mxfp8")
    single = _gemm(hq, aq, bq, sfa, sfb, "w8a8-mxfp8")
    monkeypatch.setenv("HALOPS_B200_TILE", "pair256")
    assert "pair=1" in hq.describe_tile(m, n, k, "w8a8-mxfp8")
    out = torch.empty_like(single)
    different = torch.zeros([], dtype=torch.int64, device="cuda")
    for _ in range(200):
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, "w8a8-mxfp8", True)
        different += (out.view(torch.int16) != single.view(torch.int16)).any()
    assert hq.device_status() == 0
    assert int(different) == 0, f"{int(different)} of 200 runs differ from the single-CTA tile"


@pytest.mark.parametrize("m,n,k", [(1344, 16384, 1024), (100, 7168, 512)])
def test_no_out_of_bounds_write(hq, m, n, k):
    """The output is a view of a larger sentinel-filled buffer; bytes past the
    view stay untouched (reference tests/test_dense_gemm.py:308-329)."""
    a, b = _rand(m, k, 11), _rand(n, k, 12)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    guard, sentinel = 128, 0x5A
    buf = torch.full([(m + guard) * n * 2], sentinel, dtype=torch.uint8, device="cuda")
    out = buf[: m * n * 2].view(torch.bfloat16).view(m, n)
    hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, "w8a8-mxfp8", True)
    torch.cuda.synchronize()
    assert (buf[m * n * 2:] == sentinel).all()
    _check(out, aq, bq, sfa, sfb, "w8a8-mxfp8")


def test_strided_output(hq):
    m, n, k = 192, 256, 512
    a, b = _rand(m, k, 13), _rand(n, k, 14)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    wide = torch.full([m, 3 * n], 7.0, dtype=torch.bfloat16, device="cuda")
    out = wide[:, n:2 * n]
    hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, "w8a8-mxfp8")
    torch.cuda.synchronize()
    assert (wide[:, :n] == 7.0).all() and (wide[:, 2 * n:] == 7.0).all()
    _check(out.contiguous(), aq, bq, sfa, sfb, "w8a8-mxfp8")


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4"])
def test_determinism_pdl_and_sm_count(hq, mode):
    """Bitwise identical across runs, with and without PDL, and for any SM count."""
    a, b = _rand(1024, 2048, 15), _rand(2048, 2048, 16)
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    base = _gemm(hq, aq, bq, sfa, sfb, mode)
    assert torch.equal(base, _gemm(hq, aq, bq, sfa, sfb, mode))
    assert torch.equal(base, _gemm(hq, aq, bq, sfa, sfb, mode, use_pdl=True))
    assert torch.equal(base, _gemm(hq, aq, bq, sfa, sfb, mode, sm_count=37))
    _check(base, aq, bq, sfa, sfb, mode, alpha=1.0 if mode == "w4a4-nvfp4" else None)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-mxfp4", "w4a4-nvfp4"])
def test_pdl_chain_after_group_wise_quant(hq, mode):
    """quantize -> GEMM with PDL on both kernels and no synchronisation in
    between equals the plain chain (reference tests/test_dense_gemm.py:679-706)."""
    m, n, k = 512, 1024, 1024
    a, b = _rand(m, k, 17).cuda(), _rand(n, k, 18).cuda()
    alpha = torch.ones([1], dtype=torch.float32, device="cuda") if mode == "w4a4-nvfp4" else None
    x, sfa = hq.group_wise_quant(a, mode=mode, use_pdl=False)
    w, sfb = hq.group_wise_quant(b, mode=mode, use_pdl=False)
    ref = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(x, w, sfa, sfb, ref, None, alpha, -1, mode, False)
    for _ in range(8):
        x, sfa = hq.group_wise_quant(a, mode=mode, use_pdl=True)
        w, sfb = hq.group_wise_quant(b, mode=mode, use_pdl=True)
        out = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
        hq.dense_gemm(x, w, sfa, sfb, out, None, alpha, -1, mode, True)
        assert torch.equal(out, ref)
    assert hq.device_status() == 0


def test_end_to_end_unaligned(hq):
    """The user flow with no manual pad or slice (reference :591-611)."""
    m, n, k = 300, 1024, 2048
    a, b = _rand(m, k, 19), _rand(n, k, 20)
    x, sfa = hq.group_wise_quant(a.cuda())
    w, sfb = hq.group_wise_quant(b.cuda())
    assert list(x.shape) == [m, k] and list(sfa.shape) == [384, k // 32]
    out = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(x, w, sfa, sfb, out, None, None, -1, "w8a8-mxfp8")
    _check(out, x, w, sfa, sfb, "w8a8-mxfp8")
    # and close to the unquantised product
    ref = a.float() @ b.float().T
    rel = (out.float().cpu() - ref).norm() / ref.norm()
    assert rel < 0.05


def test_errors_on_device(hq):
    dev = "cuda"
    x = torch.empty([128, 128], dtype=torch.float8_e4m3fn, device=dev)
    w = torch.empty([256, 128], dtype=torch.float8_e4m3fn, device=dev)
    sfa = torch.empty([128, 4], dtype=torch.uint8, device=dev)
    sfb = torch.empty([256, 4], dtype=torch.uint8, device=dev)
    out = torch.empty([128, 256], dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="sfa must hold whole 128-row SfAtoms"):
        hq.dense_gemm(x, w, sfa[:64], sfb, out)
    with pytest.raises(RuntimeError, match="sfb must hold whole 128-row SfAtoms"):
        hq.dense_gemm(x, w, sfa, sfb[:128], out)
    with pytest.raises(RuntimeError, match="Unsupported epilogue"):
        hq.dense_gemm(x, w, sfa, sfb, out, epilogue=hq.EpilogueOp.Quant)
    with pytest.raises(RuntimeError, match="multiple of 256"):
        hq.dense_gemm(x, w, sfa, sfb, out, torch.zeros([256], dtype=torch.bfloat16, device=dev))


@pytest.mark.parametrize("tile", ["pair256", "pair128", "256", "128", "64"])
@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4"])
@pytest.mark.parametrize("m,n,k", [(512, 1024, 1024), (300, 512, 768), (2304, 2048, 512)], ids=lambda v: str(v))
def test_every_tile_shape(hq, monkeypatch, tile, mode, m, n, k):
    """Every compiled tile - single-CTA 128x{64,128,256} and the 2-CTA pair tiles
    256x{128,256} - gives the same result, whatever the dispatch would pick."""
    if tile == "64" and mode != "w8a8-mxfp8":
        pytest.skip("64-wide tiles exist for MXFP8 only")
    if mode != "w8a8-mxfp8" and k % 256:
        pytest.skip("FP4 modes need K % 256 == 0")
    a, b = _rand(m, k, 21), _rand(n, k, 22)
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    base = _gemm(hq, aq, bq, sfa, sfb, mode)
    monkeypatch.setenv("HALOPS_B200_TILE", tile)
    want = ("256x" if tile.startswith("pair") else "128x") + tile.replace("pair", "")
    assert want in hq.describe_tile(m, n, k, mode)
    out = _gemm(hq, aq, bq, sfa, sfb, mode)
    monkeypatch.delenv("HALOPS_B200_TILE")
    assert torch.equal(out, base), "tiles disagree bitwise"
    _check(out, aq, bq, sfa, sfb, mode, alpha=1.0 if mode == "w4a4-nvfp4" else None)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4"])
@pytest.mark.parametrize("m,n,k", [(16, 7168, 4096), (64, 4096, 512), (512, 4096, 1024), (4096, 7168, 2048)],
                         ids=lambda v: str(v))
def test_sigmoid_epilogue(hq, mode, m, n, k):
    """Reference tests/test_dense_gemm.py:215-230: sigmoid of the Identity output,
    rtol 1e-2 / atol 4e-3; also checked against the oracle's float32 product."""
    a, b = _rand(m, k, 31), _rand(n, k, 32, "weight")
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    alpha = torch.full([1], 0.8, dtype=torch.float32, device="cuda") if mode == "w4a4-nvfp4" else None
    ref = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, ref, None, alpha, -1, mode)
    out = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, out, None, alpha, -1, mode, True, hq.EpilogueOp.Sigmoid)
    assert hq.device_status() == 0
    torch.testing.assert_close(out.float(), torch.sigmoid(ref.float()), rtol=1e-2, atol=4e-3)
    if m <= 512:
        acc = oracle.dequantize(aq, sfa, mode) @ oracle.dequantize(bq, sfb, mode).T
        want = torch.sigmoid(acc * (0.8 if alpha is not None else 1.0))
        torch.testing.assert_close(out.float().cpu(), want, rtol=1e-2, atol=4e-3)


@pytest.mark.parametrize("m,n,k", [(1024, 4096, 1024), (2048, 7168, 512), (256, 256, 128)], ids=lambda v: str(v))
@pytest.mark.parametrize("tile", ["", "pair256", "128"])
def test_bias_and_sigmoid_bias(hq, monkeypatch, m, n, k, tile):
    """Bias add (bf16 [N]) in the Identity epilogue against the oracle, and the
    reference's sigmoid-with-bias check (tests/test_dense_gemm.py:233-243)."""
    if tile and n % int(tile.replace("pair", "")):
        pytest.skip("tile does not divide N")
    monkeypatch.setenv("HALOPS_B200_TILE", tile)
    a, b = _rand(m, k, 33), _rand(n, k, 34)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    bias = torch.rand([n], generator=torch.Generator().manual_seed(35)).to(torch.bfloat16).cuda()
    ref = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, ref, bias, None, -1, "w8a8-mxfp8")
    acc = oracle.dequantize(aq, sfa, "w8a8-mxfp8") @ oracle.dequantize(bq, sfb, "w8a8-mxfp8").T
    want = (acc + bias.float().cpu()).to(torch.bfloat16).float()
    torch.testing.assert_close(ref.float().cpu(), want, **W8A8_TOL)
    out = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, out, bias, None, -1, "w8a8-mxfp8", True, hq.EpilogueOp.Sigmoid)
    assert hq.device_status() == 0
    torch.testing.assert_close(out.float(), torch.sigmoid(ref.float()), rtol=1e-2, atol=8e-3)


def test_bias_rules(hq):
    a, b = _rand(200, 1024, 36), _rand(1024, 1024, 37)
    aq, bq, sfa, sfb = _quantize(hq, a, b, "w8a8-mxfp8")
    out = torch.empty([200, 1024], dtype=torch.bfloat16, device="cuda")
    bias = torch.zeros([1024], dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 256"):
        hq.dense_gemm(aq, bq, sfa, sfb, out, bias)
    aq4, bq4, sfa4, sfb4 = _quantize(hq, _rand(256, 1024, 38), b, "w4a4-mxfp4")
    with pytest.raises(RuntimeError, match="does not support bias"):
        hq.dense_gemm(aq4, bq4, sfa4, sfb4, torch.empty([256, 1024], dtype=torch.bfloat16, device="cuda"), bias,
                      None, -1, "w4a4-mxfp4")


@pytest.mark.parametrize("m, n, k, with_bias, beta, linear_beta", [
    (16, 8192, 4096, False, 4.0, 25.0), (64, 16384, 1024, False, 4.0, 25.0), (100, 4096, 512, False, 4.0, 25.0),
    (512, 4096, 1024, False, 4.0, 25.0), (4096, 7168, 2048, False, 4.0, 25.0), (1024, 4096, 1024, True, 4.0, 25.0),
    (16, 8192, 4096, True, 4.0, 25.0), (100, 4096, 512, True, 4.0, 25.0), (16, 8192, 4096, False, 2.0, None),
    (512, 4096, 1024, False, 1.0, 8.0), (200, 256, 256, True, 4.0, 25.0)], ids=lambda v: str(v))
def test_situ_quant_epilogue(hq, m, n, k, with_bias, beta, linear_beta):
    """SiTU-GLU + MXFP8 re-quantisation (reference tests/test_dense_gemm.py:250-305): the
    dequantised output is within one e4m3 step of the float32 formula, and every scale
    is the smallest power of two that keeps its group inside +-448."""
    g = torch.Generator().manual_seed(41)
    a, b = _rand(m, k, 41), _rand(n, k, 42, "weight") * 4
    aq, sfa = hq.group_wise_quant(a.cuda())
    bq, sfb_unused = hq.group_wise_quant(b.cuda())
    del sfb_unused
    bias = torch.randn([n], generator=g).to(torch.bfloat16) if with_bias else None
    # float32 reference on the dequantised operands, gate = first half of the columns
    y = oracle.dequantize(aq, sfa, "w8a8-mxfp8") @ oracle.dequantize(*hq.group_wise_quant(b.cuda()), "w8a8-mxfp8").T
    gate, up = (y + (bias.float() if with_bias else 0)).chunk(2, dim=1)
    ref = beta * torch.tanh(gate / beta) * torch.sigmoid(gate)
    ref = ref * (linear_beta * torch.tanh(up / linear_beta) if linear_beta is not None else up)
    ref = ref.to(torch.bfloat16).float()
    # kernel inputs: [gate; up] rows interleaved in blocks of 16
    w_il = hq.interleave_gate_up(b.cuda()).contiguous()
    wq, sfb = hq.group_wise_quant(w_il)
    b_il = hq.interleave_gate_up(bias.cuda()).contiguous() if with_bias else None
    q = torch.empty([m, n // 2], dtype=torch.float8_e4m3fn, device="cuda")
    kb_out = n // 2 // 32
    m_sf = (m + 127) // 128 * 128
    # not cleared by the caller: the kernel writes the zero bytes of the padding rows itself
    sf = torch.full([m_sf * kb_out], 0xAB, dtype=torch.uint8, device="cuda")
    hq.dense_gemm(aq, wq, sfa, sfb, q, b_il, None, -1, "w8a8-mxfp8", True, hq.EpilogueOp.SituQuant, sf, beta,
                  linear_beta)
    assert hq.device_status() == 0
    pad = torch.ones(sf.numel(), dtype=torch.bool)
    pad[torch.from_numpy(oracle.sf_atom_offsets(m, kb_out)).flatten()] = False
    assert (sf.cpu()[pad] == 0).all(), "padding rows of output_sf must be zero bytes"
    sf_log = torch.from_numpy(oracle.unswizzle_sf(sf.cpu().numpy().reshape(m_sf, kb_out), m))
    scale = torch.exp2(sf_log.float() - 127).repeat_interleave(32, 1)
    deq = q.float().cpu() * scale
    err = (deq - ref).abs()
    assert (err <= ref.abs() * 2 ** -3 + scale * 2 ** -9).all()
    assert (err.norm() / ref.norm()) < 0.04
    # scales: smallest power of two >= amax / 448 of what was actually stored, never too small
    amax = deq.abs().reshape(m, kb_out, 32).amax(-1)
    s = scale.reshape(m, kb_out, 32)[:, :, 0]
    assert (amax <= 448 * s).all()
    nz = ref.abs().reshape(m, kb_out, 32).amax(-1) > 1e-6
    assert (amax[nz] > 448 * s[nz] / 2 * 0.9).all(), "a scale is a step too large"


@pytest.mark.parametrize("mode, m, n, k", [
    ("w8a8-mxfp8", 1, 4096, 4096), ("w8a8-mxfp8", 64, 4096, 8192), ("w8a8-mxfp8", 128, 2048, 1024),
    ("w8a8-mxfp8", 5, 64, 2048), ("w8a8-mxfp8", 33, 4736, 1152), ("w8a8-mxfp8", 100, 1024, 1024)],
    ids=lambda v: str(v))
def test_split_k_shapes(hq, monkeypatch, mode, m, n, k):
    """One row of at most 74 64-wide tiles and at least 8 k-tiles: two CTAs share a tile, half
    of K each, partial sums through distributed shared memory.  Without the split the same tile
    runs with two MMA issuers that take alternate k-tiles into accumulators of their own.  Both
    are deterministic and within a bfloat16 rounding of each other and of the 128-wide tile
    (which sums the k-tiles in order)."""
    a, b = _rand(m, k, 21), _rand(n, k, 22, "weight")
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    monkeypatch.setenv("HALOPS_B200_TILE", "64")
    monkeypatch.setenv("HALOPS_B200_SPLITK", "0")
    assert "128x64" in hq.describe_tile(m, n, k, mode) and "splitk=0" in hq.describe_tile(m, n, k, mode)
    unsplit = _gemm(hq, aq, bq, sfa, sfb, mode)
    _check(unsplit, aq, bq, sfa, sfb, mode)
    assert torch.equal(unsplit, _gemm(hq, aq, bq, sfa, sfb, mode, use_pdl=True))
    monkeypatch.delenv("HALOPS_B200_SPLITK")
    assert "splitk=1" in hq.describe_tile(m, n, k, mode)
    out = _gemm(hq, aq, bq, sfa, sfb, mode)
    _check(out, aq, bq, sfa, sfb, mode)
    assert torch.equal(out, _gemm(hq, aq, bq, sfa, sfb, mode, use_pdl=True))

    def close(x, y):  # one bfloat16 step (2^-8 relative) plus the float32 reordering noise near zero
        diff = (x.float() - y.float()).abs()
        return bool((diff <= y.float().abs() * 2 ** -7 + 1e-3 * y.float().abs().max()).all())

    assert close(out, unsplit)
    if n % 128 == 0:
        monkeypatch.setenv("HALOPS_B200_TILE", "128")
        in_order = _gemm(hq, aq, bq, sfa, sfb, mode)
        assert close(out, in_order) and close(unsplit, in_order)


@pytest.mark.parametrize("mode, m, n, k", [("w8a8-mxfp8", 256, 512, 1024), ("w8a8-mxfp8", 100, 256, 512),
                                           ("w4a4-nvfp4", 384, 256, 512), ("w8a8-mxfp8", 1024, 2048, 1024)],
                         ids=lambda v: str(v))
def test_register_store_epilogue_equals_tma_store(hq, monkeypatch, mode, m, n, k):
    """HALOPS_B200_EPILOGUE=direct stores every tile of the single-CTA kernel from registers,
    row by row, instead of through the staging buffers and TMA stores: same bits."""
    a, b = _rand(m, k, 23), _rand(n, k, 24)
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    monkeypatch.setenv("HALOPS_B200_TILE", "128")
    staged = _gemm(hq, aq, bq, sfa, sfb, mode)
    monkeypatch.setenv("HALOPS_B200_EPILOGUE", "direct")
    direct = _gemm(hq, aq, bq, sfa, sfb, mode)
    assert hq.device_status() == 0
    assert torch.equal(staged, direct)
    _check(direct, aq, bq, sfa, sfb, mode)


@pytest.mark.parametrize("mode, m, n, k", [("w8a8-mxfp8", 2048, 2048, 4096), ("w4a4-nvfp4", 1024, 2048, 4096),
                                           ("w8a8-mxfp8", 1000, 1024, 1024)], ids=lambda v: str(v))
def test_pair_tile_is_bit_identical_and_deterministic(hq, monkeypatch, mode, m, n, k):
    """The 2-CTA kernel issues the MMAs of alternate k-tiles from two threads that hand the
    turn to each other; the MMAs must still reach the tensor core in k order.  Then the
    result equals the single-CTA tile's bit for bit, run after run."""
    a, b = _rand(m, k, 31), _rand(n, k, 32)
    aq, bq, sfa, sfb = _quantize(hq, a, b, mode)
    monkeypatch.setenv("HALOPS_B200_TILE", "256")
    single = _gemm(hq, aq, bq, sfa, sfb, mode)
    monkeypatch.setenv("HALOPS_B200_TILE", "pair256")
    assert "pair=1" in hq.describe_tile(m, n, k, mode)
    for _ in range(10):
        assert torch.equal(single, _gemm(hq, aq, bq, sfa, sfb, mode))
