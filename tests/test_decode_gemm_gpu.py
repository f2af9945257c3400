"""Small-M ("decode") dense GEMM: the operand-swapped kernel (128 weight rows as the M of the
MMA, activations as its N, 256 bytes of K per stage, units dealt evenly over the SMs with
float32 partial tiles summed in K order).  Checked against the oracle on the benchmark's
decode shapes (Student-t activations), the shapes the reference charts, ragged sizes, both
unit deals, the sigmoid epilogue and for bitwise determinism."""

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

TOL = dict(rtol=2e-2, atol=2e-3)  # the reference's MXFP8 tolerance (tests/test_dense_gemm.py)
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
        x = x / torch.sqrt(torch.randn([3, m, k], generator=g).pow(2).sum(0) / 3)
    return x.to(torch.bfloat16)


def _run(hq, aq, bq, sfa, sfb, **kw):
    out = torch.full([aq.shape[0], bq.shape[0]], 7.0, dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, kw.get("sm_count", -1), "w8a8-mxfp8", kw.get("use_pdl", False),
                  kw.get("epilogue", hq.EpilogueOp.Identity))
    assert hq.device_status() == 0
    return out


def _check(out, aq, bq, sfa, sfb, sigmoid=False):
    ref = oracle.dequantize(aq, sfa, "w8a8-mxfp8") @ oracle.dequantize(bq, sfb, "w8a8-mxfp8").T
    if sigmoid:
        ref = torch.sigmoid(ref)
    got = out.float().cpu()
    torch.testing.assert_close(got, ref.to(torch.bfloat16).float(), **TOL)
    rel = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert rel <= MAX_REL, f"max relative error {rel}"


def _quant(hq, a, b):
    aq, sfa = hq.group_wise_quant(a.cuda())
    bq, sfb = hq.group_wise_quant(b.cuda())
    return aq, bq, sfa, sfb


C3 = [(m, n, k) for (n, k) in ((7168, 2048), (24576, 1536)) for m in (1, 8, 32, 64, 128)]


@pytest.mark.parametrize("m,n,k", C3, ids=lambda v: str(v))
def test_benchmark_decode_shapes(hq, monkeypatch, m, n, k):
    """M in {1, 8, 32, 64, 128} x (N=7168, K=2048 | N=24576, K=1536), Student-t(3)
    activations with outlier blocks, N(0, 0.02) weights.  Up to 64 rows go to the
    operand-swapped kernel by default; 128 rows are sent there too for this test."""
    if m > 64:
        assert "swap" not in hq.describe_tile(m, n, k)
        monkeypatch.setenv("HALOPS_B200_DECODE", "wide")
    assert "swap" in hq.describe_tile(m, n, k)
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 100 + m, "student_t"), _rand(n, k, 200 + m, "weight"))
    _check(_run(hq, aq, bq, sfa, sfb), aq, bq, sfa, sfb)


@pytest.mark.parametrize("m,n,k", [(8, 8192, 1024), (64, 8192, 1024), (8, 32768, 1024), (32, 8192, 4096),
                                   (128, 8192, 4096), (64, 4096, 8192), (128, 4096, 8192), (128, 256, 512)],
                         ids=lambda v: str(v))
@pytest.mark.parametrize("wide", [False, True], ids=["default", "wide"])
def test_charted_shapes(hq, monkeypatch, m, n, k, wide):
    """The small-M shapes of the reference's performance chart and its CI case 128 x 256 x 512,
    as the dispatch sends them and with every one of them on the operand-swapped kernel."""
    if wide:
        monkeypatch.setenv("HALOPS_B200_DECODE", "wide")
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 300 + m), _rand(n, k, 400 + m))
    _check(_run(hq, aq, bq, sfa, sfb), aq, bq, sfa, sfb)


@pytest.mark.parametrize("m,n,k", [(1, 64, 128), (5, 192, 384), (17, 4736, 1152), (33, 128, 128), (100, 1024, 1024),
                                   (127, 320, 640), (16, 64, 4096), (9, 2112, 256), (128, 128, 8192)],
                         ids=lambda v: str(v))
@pytest.mark.parametrize("deal", ["wide", "wide,split", "wide,split,nocluster", "wide,nosplit"])
def test_ragged_sizes_and_both_deals(hq, monkeypatch, m, n, k, deal):
    """M off the activation widths, N with a last tile of 64 rows, K with a last step of 128
    bytes, one tile, one step; with every tile dealt to several CTAs where there are SMs for
    that (partial tiles through the first CTA's shared memory in a cluster, or through the
    scratch buffer), with whole tiles per CTA, and as the dispatch decides.  Rows past M and columns past N
    are never written (the output is a window of a sentinel-filled buffer)."""
    monkeypatch.setenv("HALOPS_B200_DECODE", deal)
    assert "swap" in hq.describe_tile(m, n, k)
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 500 + m), _rand(n, k, 600 + m))
    guard = torch.full([m + 2, n + 16], 3.0, dtype=torch.bfloat16, device="cuda")
    out = guard[1:m + 1, 8:n + 8]
    hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, "w8a8-mxfp8", False)
    assert hq.device_status() == 0
    _check(out.contiguous(), aq, bq, sfa, sfb)
    guard[1:m + 1, 8:n + 8] = 3.0
    assert (guard == 3.0).all(), "wrote outside the [M, N] window"


@pytest.mark.parametrize("m,n,k", [(8, 7168, 2048), (128, 4096, 2048), (64, 4096, 8192), (16, 640, 1152)],
                         ids=lambda v: str(v))
@pytest.mark.parametrize("exchange", ["cluster", "scratch"])
def test_deterministic_and_pdl(hq, monkeypatch, m, n, k, exchange):
    """Partial tiles are summed in K order, not in arrival order: 30 runs give the same bits,
    with and without programmatic launch, whether they are exchanged through shared memory
    in a cluster or through the scratch buffer; a split and an unsplit run differ only by
    float32 reassociation."""
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 700 + m, "student_t"), _rand(n, k, 800 + m, "weight"))
    monkeypatch.setenv("HALOPS_B200_DECODE", "wide,split" + (",nocluster" if exchange == "scratch" else ""))
    tile = hq.describe_tile(m, n, k)
    assert "splitk=1" in tile and ("cluster=1" in tile) == (exchange == "scratch")
    base = _run(hq, aq, bq, sfa, sfb)
    _check(base, aq, bq, sfa, sfb)
    for i in range(30):
        assert torch.equal(base, _run(hq, aq, bq, sfa, sfb, use_pdl=bool(i & 1))), f"run {i} differs"
    monkeypatch.setenv("HALOPS_B200_DECODE", "wide,nosplit")
    assert "splitk=0" in hq.describe_tile(m, n, k)
    whole = _run(hq, aq, bq, sfa, sfb)
    _check(whole, aq, bq, sfa, sfb)
    diff = (whole.float() - base.float()).abs()
    assert (diff <= whole.float().abs() * 2 ** -7 + 1e-3 * whole.float().abs().max()).all()


def test_back_to_back_launches_share_the_scratch_buffer(hq, monkeypatch):
    """Two different split problems queued on one stream without a synchronisation in between
    use the same scratch buffer and tile counters one after the other."""
    monkeypatch.setenv("HALOPS_B200_DECODE", "wide,split,nocluster")
    p1 = _quant(hq, _rand(8, 2048, 1), _rand(7168, 2048, 2, "weight"))
    p2 = _quant(hq, _rand(100, 1536, 3), _rand(4736, 1536, 4, "weight"))
    o1 = torch.empty([8, 7168], dtype=torch.bfloat16, device="cuda")
    o2 = torch.empty([100, 4736], dtype=torch.bfloat16, device="cuda")
    assert "splitk=1" in hq.describe_tile(8, 7168, 2048) and "splitk=1" in hq.describe_tile(100, 4736, 1536)
    for _ in range(5):
        hq.dense_gemm(p1[0], p1[1], p1[2], p1[3], o1)
        hq.dense_gemm(p2[0], p2[1], p2[2], p2[3], o2)
    assert hq.device_status() == 0
    _check(o1, *p1)
    _check(o2, *p2)


def test_second_stream_gets_its_own_scratch(hq, monkeypatch):
    monkeypatch.setenv("HALOPS_B200_DECODE", "split,nocluster")
    p1 = _quant(hq, _rand(16, 2048, 5), _rand(7168, 2048, 6, "weight"))
    want = _run(hq, *p1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    outs = []
    with torch.cuda.stream(side):
        for _ in range(3):
            o = torch.empty_like(want)
            hq.dense_gemm(p1[0], p1[1], p1[2], p1[3], o)
            outs.append(o)
    for _ in range(3):
        o = torch.empty_like(want)
        hq.dense_gemm(p1[0], p1[1], p1[2], p1[3], o)
        outs.append(o)
    torch.cuda.synchronize()
    assert hq.device_status() == 0
    assert all(torch.equal(o, want) for o in outs)


@pytest.mark.parametrize("m,n,k", [(8, 1024, 1024), (100, 7168, 2048)], ids=lambda v: str(v))
def test_sigmoid_epilogue(hq, m, n, k):
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 900 + m), _rand(n, k, 901 + m, "weight") * 8)
    out = _run(hq, aq, bq, sfa, sfb, epilogue=hq.EpilogueOp.Sigmoid)
    ref = torch.sigmoid(oracle.dequantize(aq, sfa, "w8a8-mxfp8") @ oracle.dequantize(bq, sfb, "w8a8-mxfp8").T)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-2, atol=1e-2)


def test_fewer_sms_and_the_older_tile_agree(hq, monkeypatch):
    """sm_count caps the grid; HALOPS_B200_DECODE=off sends the shape to the 128 x 64 tile with
    the activations as the M of the MMA: same result within the comparison tolerance."""
    m, n, k = 32, 7168, 2048
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 11), _rand(n, k, 12, "weight"))
    _check(_run(hq, aq, bq, sfa, sfb, sm_count=37), aq, bq, sfa, sfb)
    new = _run(hq, aq, bq, sfa, sfb)
    monkeypatch.setenv("HALOPS_B200_DECODE", "off")
    assert "128x64" in hq.describe_tile(m, n, k)
    old = _run(hq, aq, bq, sfa, sfb)
    _check(old, aq, bq, sfa, sfb)
    diff = (new.float() - old.float()).abs()
    assert (diff <= old.float().abs() * 2 ** -7 + 1e-3 * old.float().abs().max()).all()


@pytest.mark.parametrize("m,n,k,env", [(128, 7168, 2048, ""), (100, 24576, 1536, ""), (65, 8192, 4096, ""),
                                       (128, 192, 256, ""), (128, 320, 128, ""), (8, 7168, 2048, "off"),
                                       (64, 4736, 1152, "off")], ids=lambda v: str(v))
def test_one_row_of_64_wide_tiles_with_two_issuers(hq, monkeypatch, m, n, k, env):
    """65 to 128 activation rows (and fewer with the small-M kernel switched off) run on the
    128 x 64 tile with the activations as the M of the MMA, where two threads issue the MMAs of
    alternate k-tiles into accumulators of their own: against the oracle, 20 runs bit-identical,
    with and without programmatic launch, plain and sigmoid epilogue, a single k-tile too."""
    if env:
        monkeypatch.setenv("HALOPS_B200_DECODE", env)
    assert "128x64/128" in hq.describe_tile(m, n, k)
    aq, bq, sfa, sfb = _quant(hq, _rand(m, k, 40 + m, "student_t"), _rand(n, k, 41 + m, "weight"))
    base = _run(hq, aq, bq, sfa, sfb)
    _check(base, aq, bq, sfa, sfb)
    for i in range(20):
        assert torch.equal(base, _run(hq, aq, bq, sfa, sfb, use_pdl=bool(i & 1))), f"run {i} differs"
    sig = _run(hq, aq, bq, sfa, sfb, epilogue=hq.EpilogueOp.Sigmoid)
    ref = torch.sigmoid(oracle.dequantize(aq, sfa, "w8a8-mxfp8") @ oracle.dequantize(bq, sfb, "w8a8-mxfp8").T)
    torch.testing.assert_close(sig.float().cpu(), ref, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("m,n,k,deal", [(8, 7168, 2048, ""), (64, 4096, 8192, ""), (16, 1024, 8192, "split,nocluster"),
                                        (1, 24576, 1536, ""), (32, 2048, 4096, "split")], ids=lambda v: str(v))
def test_chain_with_early_weight_loads(hq, monkeypatch, m, n, k, deal):
    """use_pdl=2: the weight of the first stages is asked for before the preceding kernel is known to be
    complete.  A chain of GEMMs on different weights, each reading the activation that a kernel just
    before it wrote, gives the bits of the plain launches."""
    monkeypatch.setenv("HALOPS_B200_DECODE", deal)
    g = torch.Generator().manual_seed(77 + m)
    layers = 6
    xs = [torch.randn([m, k], generator=g).to(torch.bfloat16).cuda() for _ in range(layers)]
    ws = [hq.group_wise_quant((torch.randn([n, k], generator=g) * 0.05).to(torch.bfloat16).cuda()) for _ in range(layers)]
    outs = {}
    xq = [torch.empty([m, k], dtype=torch.float8_e4m3fn, device="cuda") for _ in range(layers)]
    sfa = [torch.empty([128, k // 32], dtype=torch.uint8, device="cuda") for _ in range(layers)]
    for use_pdl in (0, 1, 2):
        res = [torch.full([m, n], 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(layers)]
        torch.cuda.synchronize()
        for _ in range(3):  # a few rounds: the scratch memory and the tile counters are reused
            for i in range(layers):
                # only this library's kernels on the stream: the quantizer writes the activation that the
                # GEMM right behind it reads, and the next quantizer follows that GEMM
                hq.group_wise_quant(xs[i], "w8a8-mxfp8", True, bool(use_pdl), xq[i], sfa[i])
                hq.dense_gemm(xq[i], ws[i][0], sfa[i], ws[i][1], res[i], None, None, -1, "w8a8-mxfp8", use_pdl)
        torch.cuda.synchronize()
        assert hq.device_status() == 0
        outs[use_pdl] = res
    for i in range(layers):
        assert torch.equal(outs[0][i], outs[1][i]) and torch.equal(outs[0][i], outs[2][i]), f"GEMM {i} of the chain differs"
