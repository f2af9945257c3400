"""GPU parity tests of ``group_masked_gemm`` and ``group_contiguous_gemm`` against the
CPU row-wise expert oracle.  Mirrors the reference's ``tests/test_group_masked_gemm.py``
and ``tests/test_group_contiguous_gemm.py`` (shape lists with the large N x K reduced
where the oracle would take minutes, partial masks, empty experts, 64-row slots that
share a tile, per-expert bias and alpha, error texts, determinism); rows past
``masked_m`` must stay untouched.  Calls go through the Python wrappers and therefore
the C ABI.  Tolerances as for ``dense_gemm``."""

import re

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

W8A8_TOL = dict(rtol=2e-2, atol=2e-3)
W4A4_TOL = dict(rtol=5e-2, atol=5e-2)
FULL_N, FULL_K = 7168, 3584  # the reference's MoE shape (tests/test_group_masked_gemm.py:395)


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _inputs(hq, m, experts, n, k, mode, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn([m, k], generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn([experts, n, k], generator=g) * 0.05).to(torch.bfloat16).cuda()
    xq, sfa = hq.group_wise_quant(x, mode=mode)
    wq, sfb = hq.group_wise_quant(w.view(experts * n, k), mode=mode)
    return xq, wq.view(experts, n, -1), sfa, sfb.view(experts, n, -1)


def _extras(mode, experts, n, add_bias):
    alpha = (0.5 + 0.125 * torch.arange(experts, dtype=torch.float32)).cuda() if mode == "w4a4-nvfp4" else None
    bias = None
    if add_bias:
        bias = torch.rand([experts, n], generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).cuda()
    return alpha, bias


def _compare(out, ref, rows, mode, bias):
    tol = dict(W8A8_TOL if mode == "w8a8-mxfp8" else W4A4_TOL)
    if bias is not None:
        tol["atol"] = 1e-2
    rows = torch.from_numpy(rows)
    torch.testing.assert_close(out.float().cpu()[rows], ref.float()[rows], **tol)


def _masked_case(hq, max_m, experts, n, k, mode, masked, add_bias=False, check_rows=None):
    xq, wq, sfa, sfb = _inputs(hq, experts * max_m, experts, n, k, mode)
    alpha, bias = _extras(mode, experts, n, add_bias)
    masked_t = torch.tensor(masked, dtype=torch.int32).cuda()
    out = torch.full([experts * max_m, n], 3.0, dtype=torch.bfloat16, device="cuda")
    hq.group_masked_gemm(xq, wq, sfa, sfb, masked_t, out, bias, alpha, max_m, -1, mode)
    assert hq.device_status() == 0
    ids = np.full(experts * max_m, -1, dtype=np.int64)
    for e, cnt in enumerate(masked):
        ids[e * max_m:e * max_m + cnt] = e
    valid = np.nonzero(ids >= 0)[0]
    if check_rows is not None and valid.size > check_rows:
        # the full problem runs on the GPU; the oracle checks a spread of its rows
        valid = valid[np.linspace(0, valid.size - 1, check_rows).astype(np.int64)]
        sel = np.full_like(ids, -1)
        sel[valid] = ids[valid]
        ids_ref = sel
    else:
        ids_ref = ids
    ref = oracle.group_gemm_ref(xq, wq, sfa, sfb, ids_ref, mode, alpha=None if alpha is None else alpha.cpu(),
                                bias=bias)
    _compare(out, ref, valid, mode, bias)
    padding = torch.from_numpy(np.nonzero(ids < 0)[0])
    assert torch.all(out.cpu()[padding] == 3.0), "rows past masked_m were written"
    return out


@pytest.mark.parametrize("max_m,experts,n,k,masked,add_bias", [
    (128, 4, 256, 256, [17, 63, 95, 127], False),
    (128, 4, 256, 256, [128, 128, 128, 128], False),
    (128, 4, 256, 256, [128, 0, 64, 1], True),
    (64, 20, 256, 256, None, False),
    (64, 6, 128, 512, [64, 0, 3, 64, 33, 0], True),
    (256, 3, 512, 128, [256, 129, 5], False),
    (192, 3, 256, 384, [100, 192, 1], False),
    (128, 4, FULL_N, FULL_K, None, False),
    (4096, 20, 1024, 512, None, False),
], ids=lambda v: str(v) if not isinstance(v, list) else "m" + "-".join(map(str, v)))
def test_masked_mxfp8(hq, max_m, experts, n, k, masked, add_bias):
    if masked is None:
        masked = [max_m] * experts
    _masked_case(hq, max_m, experts, n, k, "w8a8-mxfp8", masked, add_bias, check_rows=1024)


@pytest.mark.parametrize("mode,k", [("w4a4-nvfp4", 256), ("w4a4-mxfp4", 512)])
@pytest.mark.parametrize("max_m,experts,n,masked", [
    (128, 4, 256, None), (128, 4, 256, [17, 63, 95, 127]), (512, 8, 256, None), (64, 20, 128, None),
    (64, 5, 128, [1, 64, 0, 40, 64])], ids=lambda v: str(v) if not isinstance(v, list) else "partial")
def test_masked_fp4(hq, mode, k, max_m, experts, n, masked):
    if masked is None:
        masked = [max_m] * experts
    _masked_case(hq, max_m, experts, n, k, mode, masked, check_rows=1024)


@pytest.mark.parametrize("tile", ["pair256", "pair128"])
@pytest.mark.parametrize("max_m,experts,n,k,masked,add_bias", [
    (256, 3, 512, 128, [256, 129, 5], False),
    (512, 4, 512, 256, [512, 300, 0, 257], True),
    (256, 5, 256, 384, [0, 256, 1, 128, 255], False),
    (1024, 6, 1024, 512, None, False),
], ids=lambda v: str(v) if not isinstance(v, list) else "m" + "-".join(map(str, v)))
def test_masked_mxfp8_on_the_2cta_tile(hq, monkeypatch, tile, max_m, experts, n, k, masked, add_bias):
    """Slots of a multiple of 256 rows run on the 2-CTA tile: full and partly filled 256-row tiles,
    empty slots, a half of a tile without valid rows; rows past masked_m stay untouched."""
    monkeypatch.setenv("HALOPS_B200_TILE", tile)
    assert "pair=1" in hq.describe_group_tile("masked", experts, max_m, n, k)
    if masked is None:
        masked = [max_m] * experts
    a = _masked_case(hq, max_m, experts, n, k, "w8a8-mxfp8", masked, add_bias, check_rows=1024)
    # the same bits as the single-CTA tiles (every kernel sums the k-tiles in order)
    monkeypatch.setenv("HALOPS_B200_TILE", "128")
    b = _masked_case(hq, max_m, experts, n, k, "w8a8-mxfp8", masked, add_bias, check_rows=1024)
    assert torch.equal(a, b)


@pytest.mark.parametrize("tile", ["pair256", "pair128"])
@pytest.mark.parametrize("counts,n,k,add_bias", [
    ([256, 256], 512, 256, False),
    ([64, 192, 128, 64, 64], 256, 128, True),          # two and three runs of experts in a 256-row tile
    ([64] * 8, 256, 256, False),                       # four experts per tile
    ([0, 128, 0, 384, 256], 256, 256, True),           # experts without rows, a run across two tiles
    ([256] * 16, 1024, 512, False),
], ids=lambda v: str(v) if not isinstance(v, list) else "runs" + "-".join(map(str, v)))
def test_contiguous_mxfp8_on_the_2cta_tile(hq, monkeypatch, tile, counts, n, k, add_bias):
    monkeypatch.setenv("HALOPS_B200_TILE", tile)
    m = int(sum(counts))
    assert m % 256 == 0
    assert "pair=1" in hq.describe_group_tile("contiguous", len(counts), m // len(counts), n, k, total_m=m)
    a = _contiguous_case(hq, counts, n, k, "w8a8-mxfp8", add_bias, check_rows=1024)
    monkeypatch.setenv("HALOPS_B200_TILE", "128")
    b = _contiguous_case(hq, counts, n, k, "w8a8-mxfp8", add_bias, check_rows=1024)
    assert torch.equal(a, b)


def test_masked_determinism_and_sm_count(hq):
    xq, wq, sfa, sfb = _inputs(hq, 6 * 128, 6, 256, 256, "w8a8-mxfp8", seed=2)
    masked = torch.tensor([128, 5, 0, 77, 128, 64], dtype=torch.int32).cuda()
    outs = []
    for sm in (-1, -1, 5, 148):
        out = torch.zeros([6 * 128, 256], dtype=torch.bfloat16, device="cuda")
        hq.group_masked_gemm(xq, wq, sfa, sfb, masked, out, None, None, 128, sm)
        outs.append(out)
    assert hq.device_status() == 0
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def _spans(counts):
    return np.concatenate([np.full(c, e, dtype=np.int32) for e, c in enumerate(counts)])


def _contiguous_case(hq, counts, n, k, mode, add_bias=False, check_rows=None):
    ids = _spans(counts)
    m, experts = ids.size, len(counts)
    xq, wq, sfa, sfb = _inputs(hq, m, experts, n, k, mode, seed=4)
    alpha, bias = _extras(mode, experts, n, add_bias)
    out = torch.full([m, n], float("nan"), dtype=torch.bfloat16, device="cuda")
    hq.group_contiguous_gemm(xq, wq, sfa, sfb, torch.from_numpy(ids).cuda(), out, bias, alpha, -1, mode)
    assert hq.device_status() == 0
    rows = np.arange(m)
    ids_ref = ids.astype(np.int64)
    if check_rows is not None and m > check_rows:
        rows = np.linspace(0, m - 1, check_rows).astype(np.int64)
        ids_ref = np.full(m, -1, dtype=np.int64)
        ids_ref[rows] = ids[rows]
    ref = oracle.group_gemm_ref(xq, wq, sfa, sfb, ids_ref, mode, alpha=None if alpha is None else alpha.cpu(),
                                bias=bias)
    _compare(out, ref, rows, mode, bias)
    assert not torch.isnan(out.float()).any(), "some rows were not written"
    return out


@pytest.mark.parametrize("counts,n,k,add_bias", [
    ([256, 256], 512, 256, False),                 # m512_e2
    ([256] * 16, 1024, 512, False),                # large_m4096_e20 (16 experts fit)
    ([64] * 1, 256, 256, False),                   # small_m64
    ([64] * 20, 256, 256, False),                  # 64-row runs: two experts per tile
    ([128], 256, 256, False),                      # m128_n256_k256_e1
    ([64, 192, 128, 64, 64, 320], 256, 128, True),  # runs that start mid-tile
    ([0, 128, 0, 64], 128, 256, True),             # experts without rows
    ([256, 256], FULL_N, FULL_K, False),
], ids=lambda v: str(v) if not isinstance(v, list) else "runs" + str(len(v)))
def test_contiguous_mxfp8(hq, counts, n, k, add_bias):
    _contiguous_case(hq, counts, n, k, "w8a8-mxfp8", add_bias, check_rows=1024)


@pytest.mark.parametrize("mode", ["w4a4-nvfp4", "w4a4-mxfp4"])
@pytest.mark.parametrize("counts,n,k", [([256, 256], 256, 512), ([256] * 8, 512, 512), ([128], 256, 512),
                                        ([64, 64, 128, 64], 128, 512)],
                         ids=lambda v: str(v) if not isinstance(v, list) else "runs" + str(len(v)))
def test_contiguous_fp4(hq, mode, counts, n, k):
    _contiguous_case(hq, counts, n, k, mode, check_rows=1024)


def test_contiguous_equals_masked_and_dense(hq):
    """Same kernel, same tile, same k order: bit-equal across the three faces."""
    experts, rows, n, k = 3, 128, 256, 256
    xq, wq, sfa, sfb = _inputs(hq, experts * rows, experts, n, k, "w8a8-mxfp8", seed=6)
    ids = torch.from_numpy(_spans([rows] * experts)).cuda()
    a = torch.empty([experts * rows, n], dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(a)
    hq.group_contiguous_gemm(xq, wq, sfa, sfb, ids, a)
    hq.group_masked_gemm(xq, wq, sfa, sfb, torch.full([experts], rows, dtype=torch.int32).cuda(), b, None, None, rows)
    assert torch.equal(a, b)
    sfa_e = sfa.view(experts, rows, -1)
    for e in range(experts):
        d = torch.empty([rows, n], dtype=torch.bfloat16, device="cuda")
        hq.dense_gemm(xq[e * rows:(e + 1) * rows], wq[e], sfa_e[e].contiguous(), sfb[e].contiguous(), d)
        assert torch.equal(d, a[e * rows:(e + 1) * rows])
    assert hq.device_status() == 0


def _masked_empty(experts=2, max_m=128, n=256, k=128, device="cuda", **over):
    t = dict(
        x=torch.empty([experts * max_m, k], dtype=torch.float8_e4m3fn, device=device),
        w=torch.empty([experts, n, k], dtype=torch.float8_e4m3fn, device=device),
        sfa=torch.empty([(experts * max_m + 127) // 128 * 128, k // 32], dtype=torch.uint8, device=device),
        sfb=torch.empty([experts, n, k // 32], dtype=torch.uint8, device=device),
        masked_m=torch.full([experts], max_m, dtype=torch.int32, device=device),
        out=torch.empty([experts * max_m, n], dtype=torch.bfloat16, device=device),
    )
    t.update(over)
    return t


def test_masked_errors(hq):
    """tests/test_group_masked_gemm.py:770-866."""
    t = _masked_empty(max_m=129)
    with pytest.raises(RuntimeError, match=re.escape("No masked w8a8-mxfp8 tile for M=129")):
        hq.group_masked_gemm(t["x"], t["w"], t["sfa"], t["sfb"], t["masked_m"], t["out"], None, None, 129)
    t = _masked_empty()
    with pytest.raises(RuntimeError, match="max_m_per_expert must be greater than 0"):
        hq.group_masked_gemm(t["x"][:0], t["w"], t["sfa"], t["sfb"], t["masked_m"], t["out"][:0], None, None, 0)
    with pytest.raises(RuntimeError, match="masked_m must have dtype torch.int32"):
        hq.group_masked_gemm(t["x"], t["w"], t["sfa"], t["sfb"], t["masked_m"].long(), t["out"], None, None, 128)
    with pytest.raises(RuntimeError, match="output must be a 2D tensor"):
        hq.group_masked_gemm(t["x"], t["w"], t["sfa"], t["sfb"], t["masked_m"], t["out"].unsqueeze(-1), None, None,
                             128)
    with pytest.raises(RuntimeError, match="input M must equal num_experts"):
        hq.group_masked_gemm(t["x"], t["w"], t["sfa"], t["sfb"], t["masked_m"], t["out"], None, None, 64)
    # W4A4 rules
    experts, max_m, n, k = 2, 128, 128, 512
    x = torch.empty([experts * max_m, k // 2], dtype=torch.uint8, device="cuda")
    w = torch.empty([experts, n, k // 2], dtype=torch.uint8, device="cuda")
    sfa = torch.empty([experts * max_m, k // 16], dtype=torch.uint8, device="cuda")
    sfb = torch.empty([experts, n, k // 16], dtype=torch.uint8, device="cuda")
    out = torch.empty([experts * max_m, n], dtype=torch.bfloat16, device="cuda")
    masked = torch.full([experts], max_m, dtype=torch.int32, device="cuda")
    alpha = torch.ones([experts], dtype=torch.float32, device="cuda")
    bias = torch.empty([experts, n], dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="W4A4 mode does not support bias yet"):
        hq.group_masked_gemm(x, w, sfa, sfb, masked, out, bias, alpha, max_m, -1, "w4a4-nvfp4")
    with pytest.raises(RuntimeError, match=re.escape("requires alpha input (per-expert scaling factor)")):
        hq.group_masked_gemm(x, w, sfa, sfb, masked, out, None, None, max_m, -1, "w4a4-nvfp4")
    sfa32, sfb32 = sfa[:, : k // 32].contiguous(), sfb[:, :, : k // 32].contiguous()
    with pytest.raises(RuntimeError, match="does not take alpha"):
        hq.group_masked_gemm(x, w, sfa32, sfb32, masked, out, None, alpha, max_m, -1, "w4a4-mxfp4")


def test_contiguous_errors(hq):
    """tests/test_group_contiguous_gemm.py:579-652."""
    def tensors(m=128, n=256, k=128, experts=1):
        return (torch.empty([m, k], dtype=torch.float8_e4m3fn, device="cuda"),
                torch.empty([experts, n, k], dtype=torch.float8_e4m3fn, device="cuda"),
                torch.empty([(m + 127) // 128 * 128, k // 32], dtype=torch.uint8, device="cuda"),
                torch.empty([experts, n, k // 32], dtype=torch.uint8, device="cuda"),
                torch.zeros([m], dtype=torch.int32, device="cuda"),
                torch.empty([m, n], dtype=torch.bfloat16, device="cuda"))

    x, w, sfa, sfb, ids, out = tensors(m=129)
    with pytest.raises(RuntimeError, match=re.escape("No contiguous w8a8-mxfp8 tile for M=129")):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids, out)
    x, w, sfa, sfb, ids, out = tensors()
    with pytest.raises(RuntimeError, match="expert_ids must have dtype torch.int32"):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids.long(), out)
    with pytest.raises(RuntimeError, match="output must be a 2D tensor"):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids, out.unsqueeze(-1))
    with pytest.raises(RuntimeError, match=re.escape("expert_ids shape must be [M], got 64, expected 128")):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids[:64], out)
    with pytest.raises(RuntimeError, match="Unsupported mode: w2a2"):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids, out, None, None, -1, "w2a2")


def _bf16_from_bits(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def _golden_operands(d, mode):
    x, w = torch.from_numpy(d["x"]).cuda(), torch.from_numpy(d["w"]).cuda()
    if mode == "w8a8-mxfp8":
        x, w = x.view(torch.float8_e4m3fn), w.view(torch.float8_e4m3fn)
    elif mode == "w4a8-mxfp4":
        x = x.view(torch.float8_e4m3fn)
    alpha = torch.from_numpy(d["alpha"]).cuda() if "alpha" in d else None
    bias = _bf16_from_bits(d["bias_bits"]).cuda() if "bias_bits" in d else None
    return x, w, torch.from_numpy(d["sfa"]).cuda(), torch.from_numpy(d["sfb"]).cuda(), alpha, bias


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a8-mxfp4"])
def test_masked_golden_fixture(hq, golden_dir, mode):
    """Inputs and outputs of the reference's own input builders and CPU model
    (tests/golden/make_golden.py): partly filled, full and empty slots, per-expert alpha."""
    import os

    d = np.load(os.path.join(golden_dir, f"masked_{mode}.npz"))
    x, w, sfa, sfb, alpha, bias = _golden_operands(d, mode)
    masked = d["masked_m"]
    max_m = x.shape[0] // masked.size
    out = torch.full([x.shape[0], w.shape[1]], 3.0, dtype=torch.bfloat16, device="cuda")
    hq.group_masked_gemm(x, w, sfa, sfb, torch.from_numpy(masked).cuda(), out, bias, alpha, max_m, -1, mode)
    assert hq.device_status() == 0
    ref = _bf16_from_bits(d["out_bits"]).float()
    rows = np.concatenate([np.arange(e * max_m, e * max_m + c) for e, c in enumerate(masked)])
    _compare(out, ref, rows, "w4a4-mxfp4" if mode == "w4a8-mxfp4" else mode, bias)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4", "w4a8-mxfp4"])
def test_contiguous_golden_fixture(hq, golden_dir, mode):
    import os

    d = np.load(os.path.join(golden_dir, f"contiguous_{mode}.npz"))
    x, w, sfa, sfb, alpha, bias = _golden_operands(d, mode)
    out = torch.empty([x.shape[0], w.shape[1]], dtype=torch.bfloat16, device="cuda")
    hq.group_contiguous_gemm(x, w, sfa, sfb, torch.from_numpy(d["expert_ids"]).cuda(), out, bias, alpha, -1, mode)
    assert hq.device_status() == 0
    _compare(out, _bf16_from_bits(d["out_bits"]).float(), np.arange(x.shape[0]),
             "w4a4-mxfp4" if mode == "w4a8-mxfp4" else mode, bias)


def _inputs_w4a8(hq, m, experts, n, k, seed=0):
    """float8_e4m3fn activations (MXFP8 recipe) x packed e2m1 weights (MXFP4 recipe)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn([m, k], generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn([experts, n, k], generator=g) * 0.05).to(torch.bfloat16).cuda()
    xq, sfa = hq.group_wise_quant(x, mode="w8a8-mxfp8")
    wq, sfb = hq.group_wise_quant(w.view(experts * n, k), mode="w4a4-mxfp4")
    return xq, wq.view(experts, n, -1), sfa, sfb.view(experts, n, -1)


@pytest.mark.parametrize("max_m,experts,n,k,masked", [
    (128, 2, 256, 256, None), (64, 8, 256, 512, None), (128, 4, 256, 256, [17, 63, 0, 127]),
    (128, 4, 1024, 2048, None), (256, 3, 512, 1024, [256, 100, 7])],
    ids=lambda v: str(v) if not isinstance(v, list) else "partial")
def test_masked_w4a8(hq, max_m, experts, n, k, masked):
    """tests/test_group_masked_gemm.py:636-680: FP8 activations x MXFP4 weights."""
    masked = [max_m] * experts if masked is None else masked
    xq, wq, sfa, sfb = _inputs_w4a8(hq, experts * max_m, experts, n, k)
    out = torch.full([experts * max_m, n], 3.0, dtype=torch.bfloat16, device="cuda")
    hq.group_masked_gemm(xq, wq, sfa, sfb, torch.tensor(masked, dtype=torch.int32).cuda(), out, None, None, max_m, -1,
                         "w4a8-mxfp4")
    assert hq.device_status() == 0
    ids = np.full(experts * max_m, -1, dtype=np.int64)
    for e, cnt in enumerate(masked):
        ids[e * max_m:e * max_m + cnt] = e
    ref = oracle.group_gemm_ref(xq, wq, sfa, sfb, ids, "w4a8-mxfp4")
    _compare(out, ref, np.nonzero(ids >= 0)[0], "w4a4-mxfp4", None)
    assert torch.all(out.cpu()[torch.from_numpy(np.nonzero(ids < 0)[0])] == 3.0)


@pytest.mark.parametrize("counts,n,k", [([128, 128], 256, 256), ([64, 192, 128, 64], 256, 512), ([256] * 4, 512, 1024)],
                         ids=lambda v: str(v) if not isinstance(v, list) else "runs" + str(len(v)))
def test_contiguous_w4a8(hq, counts, n, k):
    ids = _spans(counts)
    xq, wq, sfa, sfb = _inputs_w4a8(hq, ids.size, len(counts), n, k, seed=3)
    out = torch.full([ids.size, n], float("nan"), dtype=torch.bfloat16, device="cuda")
    hq.group_contiguous_gemm(xq, wq, sfa, sfb, torch.from_numpy(ids).cuda(), out, None, None, -1, "w4a8-mxfp4")
    assert hq.device_status() == 0
    ref = oracle.group_gemm_ref(xq, wq, sfa, sfb, ids.astype(np.int64), "w4a8-mxfp4")
    _compare(out, ref, np.arange(ids.size), "w4a4-mxfp4", None)


@pytest.mark.parametrize("tile", ["pair256", "pair128"])
def test_w4a8_on_the_2cta_tile(hq, monkeypatch, tile):
    """FP8 activations x MXFP4 weights on the 2-CTA tile (slots / M of a multiple of 256 rows): against the
    oracle and bit for bit against the single-CTA tile."""
    def masked_run():
        max_m, experts, n, k, masked = 256, 3, 512, 1024, [256, 100, 7]
        xq, wq, sfa, sfb = _inputs_w4a8(hq, experts * max_m, experts, n, k)
        out = torch.full([experts * max_m, n], 3.0, dtype=torch.bfloat16, device="cuda")
        hq.group_masked_gemm(xq, wq, sfa, sfb, torch.tensor(masked, dtype=torch.int32).cuda(), out, None, None, max_m,
                             -1, "w4a8-mxfp4")
        ids = np.full(experts * max_m, -1, dtype=np.int64)
        for e, cnt in enumerate(masked):
            ids[e * max_m:e * max_m + cnt] = e
        return out, (xq, wq, sfa, sfb), ids

    def contiguous_run():
        counts, n, k = [64, 192, 256, 128, 128], 512, 1024
        ids = _spans(counts)
        xq, wq, sfa, sfb = _inputs_w4a8(hq, ids.size, len(counts), n, k, seed=3)
        out = torch.full([ids.size, n], float("nan"), dtype=torch.bfloat16, device="cuda")
        hq.group_contiguous_gemm(xq, wq, sfa, sfb, torch.from_numpy(ids).cuda(), out, None, None, -1, "w4a8-mxfp4")
        return out, (xq, wq, sfa, sfb), ids.astype(np.int64)

    for run, kind, args in ((masked_run, "masked", (3, 256, 512, 1024)), (contiguous_run, "contiguous", (5, 153, 512, 1024))):
        monkeypatch.setenv("HALOPS_B200_TILE", tile)
        assert "pair=1" in hq.describe_group_tile(kind, *args, mode="w4a8-mxfp4", total_m=768)
        out, ops, ids = run()
        assert hq.device_status() == 0
        ref = oracle.group_gemm_ref(*ops, ids, "w4a8-mxfp4")
        _compare(out, ref, np.nonzero(ids >= 0)[0], "w4a4-mxfp4", None)
        if kind == "masked":
            assert torch.all(out.cpu()[torch.from_numpy(np.nonzero(ids < 0)[0])] == 3.0)
        monkeypatch.setenv("HALOPS_B200_TILE", "128")
        assert torch.equal(out, run()[0])


def test_w4a8_rules(hq):
    """tests/test_group_masked_gemm.py:727-768."""
    experts, max_m, n, k = 2, 128, 256, 256
    xq, wq, sfa, sfb = _inputs_w4a8(hq, experts * max_m, experts, n, k)
    out = torch.empty([experts * max_m, n], dtype=torch.bfloat16, device="cuda")
    masked = torch.full([experts], max_m, dtype=torch.int32, device="cuda")
    bias = torch.zeros([experts, n], dtype=torch.bfloat16, device="cuda")
    alpha = torch.ones([experts], dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="W4A8 mode does not support bias"):
        hq.group_masked_gemm(xq, wq, sfa, sfb, masked, out, bias, None, max_m, -1, "w4a8-mxfp4")
    with pytest.raises(RuntimeError, match="W4A8 mode does not take alpha"):
        hq.group_masked_gemm(xq, wq, sfa, sfb, masked, out, None, alpha, max_m, -1, "w4a8-mxfp4")
    with pytest.raises(RuntimeError, match="W4A8 input K"):
        hq.group_masked_gemm(xq[:, :128].contiguous(), wq, sfa, sfb, masked, out, None, None, max_m, -1, "w4a8-mxfp4")
    with pytest.raises(RuntimeError, match="requires SF K = 8"):
        hq.group_masked_gemm(xq, wq, sfa, sfb[:, :, :4].contiguous(), masked, out, None, None, max_m, -1, "w4a8-mxfp4")
