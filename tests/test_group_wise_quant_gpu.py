"""GPU parity tests of ``group_wise_quant`` against the CPU oracle: bit-exact
quantised bytes and scale bytes.  Mirrors the reference's
``tests/test_group_wise_quant.py`` (shapes, edge cases, PDL, strided input),
calling through the Python wrapper and therefore the C ABI."""

import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

MODES = ("w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4")
GROUP = {"w8a8-mxfp8": 32, "w4a4-nvfp4": 16, "w4a4-mxfp4": 32}
# the reference's shape list (tests/test_group_wise_quant.py:268-279)
SWIZZLE_CASES = [(128, 1024), (256, 2048), (512, 3584), (1024, 4096), (2048, 7168), (4096, 3584)]
LINEAR_ONLY_CASES = [(64, 1024), (192, 2048), (320, 3584)]


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _rand(m, k, seed=2026, kind="normal", dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn([m, k], generator=g)
    if kind == "weight":
        x = x * 0.02
    elif kind == "student_t":  # df = 3: heavy tails, outlier blocks
        chi2 = torch.randn([3, m, k], generator=g).pow(2).sum(0)
        x = x / torch.sqrt(chi2 / 3)
    return x.to(dtype)


def _run(hq, x, mode, use_swizzle=True, **kw):
    q, sf = hq.group_wise_quant(x.cuda(), mode=mode, use_swizzle=use_swizzle, **kw)
    torch.cuda.synchronize()
    return q.view(torch.uint8).cpu().numpy(), sf.cpu().numpy()


def _assert_equal(got, want, what):
    if not np.array_equal(got, want):
        bad = np.argwhere(got != want)
        raise AssertionError(
            f"{what}: {len(bad)} of {got.size} bytes differ; first at {bad[0].tolist()}: "
            f"got {got[tuple(bad[0])]:#x} want {want[tuple(bad[0])]:#x}")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m,k", SWIZZLE_CASES, ids=lambda v: str(v))
def test_swizzled_matches_oracle(hq, mode, m, k):
    x = _rand(m, k)
    q, sf = _run(hq, x, mode)
    oq, osf = oracle.quant_group_wise(x, mode, use_swizzle=True)
    _assert_equal(q, oq, f"{mode} {m}x{k} codes")
    _assert_equal(sf, osf, f"{mode} {m}x{k} swizzled scales")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("m,k", SWIZZLE_CASES[:3] + LINEAR_ONLY_CASES, ids=lambda v: str(v))
def test_linear_matches_oracle(hq, mode, m, k):
    x = _rand(m, k, seed=7)
    q, sf = _run(hq, x, mode, use_swizzle=False)
    oq, osf = oracle.quant_group_wise(x, mode, use_swizzle=False)
    _assert_equal(q, oq, f"{mode} {m}x{k} codes")
    _assert_equal(sf, osf, f"{mode} {m}x{k} linear scales")


def test_large_scale_case(hq):
    """The reference's largest case, 32768 x 3584 (117 M elements)."""
    x = _rand(32768, 3584, seed=11)
    q, sf = _run(hq, x, "w8a8-mxfp8")
    oq, osf = oracle.quant_group_wise(x, "w8a8-mxfp8")
    _assert_equal(q, oq, "codes")
    _assert_equal(sf, osf, "scales")


@pytest.mark.parametrize("m,k,kind", [(16384, 8192, "normal"), (7168, 8192, "weight")], ids=lambda v: str(v))
def test_sharded_config_operands(hq, m, k, kind):
    """The operands of the N-sharded configuration at full size, bit for bit: the
    replicated 16384 x 8192 activation (N(0,1)) and one rank's 7168 x 8192 weight shard
    (N(0,0.02)) of 57344 rows over 8 GPUs."""
    x = _rand(m, k, seed=13, kind=kind)
    q, sf = _run(hq, x, "w8a8-mxfp8")
    oq, osf = oracle.quant_group_wise(x, "w8a8-mxfp8")
    _assert_equal(q, oq, "codes")
    _assert_equal(sf, osf, "scales")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("kind", ["weight", "student_t"])
def test_benchmark_distributions(hq, mode, kind):
    """N(0, 0.02) weights and Student-t(3) activations (outlier blocks)."""
    x = _rand(384, 2048, seed=5, kind=kind)
    q, sf = _run(hq, x, mode)
    oq, osf = oracle.quant_group_wise(x, mode)
    _assert_equal(q, oq, f"{mode} {kind} codes")
    _assert_equal(sf, osf, f"{mode} {kind} scales")


@pytest.mark.parametrize("mode", MODES)
def test_fp16_input(hq, mode):
    x = _rand(256, 1024, seed=3, dtype=torch.float16)
    q, sf = _run(hq, x, mode)
    oq, osf = oracle.quant_group_wise(x, mode)
    _assert_equal(q, oq, f"{mode} fp16 codes")
    _assert_equal(sf, osf, f"{mode} fp16 scales")


@pytest.mark.parametrize("mode, key, floor", [("w8a8-mxfp8", "sf_mxfp8", 1e-4),
                                             ("w4a4-nvfp4", "sf_nvfp4", 1e-10),
                                             ("w4a4-mxfp4", "sf_mxfp4", 1e-10)])
def test_every_bf16_amax(hq, golden_dir, mode, key, floor):
    """One group per finite non-negative bf16 value: the scale byte equals the
    oracle's everywhere and the reference model's wherever its amax clip is
    not active."""
    d = np.load(os.path.join(golden_dir, "amax_sweep.npz"))
    g = GROUP[mode]
    amax = torch.from_numpy(d["amax_bits"].view(np.int16)).view(torch.bfloat16)
    x = torch.zeros([amax.numel(), 4 * g], dtype=torch.bfloat16)
    x[:, 0] = amax
    x[:, g + 3] = -amax          # sign must not matter
    x[:, 2 * g + g - 1] = amax   # nor the position in the group
    q, sf = _run(hq, x, mode, use_swizzle=False)
    oq, osf = oracle.quant_group_wise(x, mode, use_swizzle=False)
    _assert_equal(sf, osf, f"{mode} scale bytes")
    _assert_equal(q, oq, f"{mode} codes")
    ok = amax.float().numpy() >= floor
    for col in range(3):
        _assert_equal(sf[ok, col], d[key][ok], f"{mode} scale bytes vs reference model, group {col}")
    # an all-zero group takes the kernel's 1e-10 floor
    assert (sf[:, 3] == osf[0, 3]).all()


@pytest.mark.parametrize("mode", MODES)
def test_every_bf16_value(hq, mode):
    """All 65536 bf16 bit patterns (NaN and infinities included) as values,
    sorted so that groups hold neighbouring magnitudes, and shuffled."""
    bits = np.arange(65536, dtype=np.uint16)
    srt = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).reshape(64, 1024)
    perm = torch.randperm(65536, generator=torch.Generator().manual_seed(1))
    shuf = srt.reshape(-1)[perm].reshape(64, 1024)
    # finite-only variant of the shuffle: groups are not poisoned by inf
    fin = shuf.clone()
    fin[~torch.isfinite(fin.float())] = 1.0
    for name, x in (("sorted", srt), ("shuffled", shuf), ("finite", fin)):
        q, sf = _run(hq, x, mode, use_swizzle=False)
        oq, osf = oracle.quant_group_wise(x, mode, use_swizzle=False)
        _assert_equal(sf, osf, f"{mode} {name} scales")
        _assert_equal(q, oq, f"{mode} {name} codes")


@pytest.mark.parametrize("m", [1, 8, 64, 127, 129, 200, 300, 1000])
def test_small_and_unaligned_m(hq, m):
    """Data keeps m rows; swizzled scales cover ceil(m/128)*128 rows with zero
    padding (reference tests/test_group_wise_quant.py:484-540)."""
    k = 1024
    x = _rand(m, k, seed=m)
    xq, sf = hq.group_wise_quant(x.cuda())
    assert list(xq.shape) == [m, k] and xq.dtype == torch.float8_e4m3fn
    assert list(sf.shape) == [(m + 127) // 128 * 128, k // 32] and sf.dtype == torch.uint8
    oq, osf = oracle.quant_group_wise(x, "w8a8-mxfp8")
    _assert_equal(xq.view(torch.uint8).cpu().numpy(), oq, "codes")
    _assert_equal(sf.cpu().numpy(), osf, "scales incl. zero padding rows")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("k", [128, 384, 1152, 2176])
def test_k_not_multiple_of_chunk(hq, mode, k):
    if GROUP[mode] == 16 and k % 64:
        pytest.skip("kb_dim % 4")
    x = _rand(130, k, seed=k)
    q, sf = _run(hq, x, mode)
    oq, osf = oracle.quant_group_wise(x, mode)
    _assert_equal(q, oq, "codes")
    _assert_equal(sf, osf, "scales")


@pytest.mark.parametrize("mode, dtype, packed_k, group", [
    ("w8a8-mxfp8", torch.float8_e4m3fn, 1024, 32),
    ("w4a4-mxfp4", torch.uint8, 512, 32),
    ("w4a4-nvfp4", torch.uint8, 512, 16)])
def test_mode_selects_dtype_and_shapes(hq, mode, dtype, packed_k, group):
    x = _rand(128, 1024).cuda()
    data, sf = hq.group_wise_quant(x, mode=mode)
    assert data.dtype == dtype and list(data.shape) == [128, packed_k]
    assert list(sf.shape) == [128, 1024 // group]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("use_swizzle", [False, True])
def test_empty_input(hq, mode, use_swizzle):
    x = torch.empty([0, 1024], dtype=torch.bfloat16, device="cuda")
    q, sf = hq.group_wise_quant(x, mode=mode, use_swizzle=use_swizzle)
    assert list(q.shape) == [0, 1024 if mode == "w8a8-mxfp8" else 512]
    assert list(sf.shape) == [0, 1024 // GROUP[mode]]


def test_errors(hq):
    x = _rand(128, 1024).cuda()
    with pytest.raises(RuntimeError, match="Unsupported quantization mode"):
        hq.group_wise_quant(x, mode="w4a4-fp6")
    with pytest.raises(RuntimeError, match="scale kb_dim must be divisible by 4"):
        hq.group_wise_quant(_rand(128, 96).cuda(), mode="w8a8-mxfp8")
    with pytest.raises(RuntimeError, match="must be a 2D tensor"):
        hq.group_wise_quant(x.reshape(2, 64, 1024))
    with pytest.raises(RuntimeError, match="bfloat16 or float16"):
        hq.group_wise_quant(x.float())
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        hq.group_wise_quant(torch.zeros([4, 1030], dtype=torch.bfloat16, device="cuda")[:, 3:1027])


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("use_swizzle", [False, True])
def test_determinism_and_pdl(hq, mode, use_swizzle):
    """Identical inputs give identical bytes; a programmatic launch changes
    when the kernel may start, never what it computes, also right after a
    kernel that produces its input."""
    src = _rand(1024, 2048, seed=9).cuda()
    plain = hq.group_wise_quant(src, mode=mode, use_swizzle=use_swizzle, use_pdl=False)
    again = hq.group_wise_quant(src, mode=mode, use_swizzle=use_swizzle, use_pdl=False)
    assert torch.equal(plain[0].view(torch.uint8), again[0].view(torch.uint8)) and torch.equal(plain[1], again[1])
    for _ in range(8):
        x = src * 2.0
        pdl = hq.group_wise_quant(x, mode=mode, use_swizzle=use_swizzle, use_pdl=True)
        ref = hq.group_wise_quant(x, mode=mode, use_swizzle=use_swizzle, use_pdl=False)
        assert torch.equal(pdl[0].view(torch.uint8), ref[0].view(torch.uint8)), "PDL read stale input"
        assert torch.equal(pdl[1], ref[1]), "PDL read stale input (scales)"


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("use_swizzle", [False, True])
@pytest.mark.parametrize("m", [1, 100, 1536])
def test_strided_input_and_preallocated_outputs(hq, mode, use_swizzle, m):
    k = 1024
    wide = _rand(m, 3 * k, seed=m + 1).cuda()
    x = wide[:, k:2 * k]
    ref, ref_sf = hq.group_wise_quant(x.contiguous(), mode=mode, use_swizzle=use_swizzle)
    out = torch.empty_like(ref)
    out_sf = torch.full_like(ref_sf, 0xFF)
    got, got_sf = hq.group_wise_quant(x, mode=mode, use_swizzle=use_swizzle, output_quant=out, output_sf=out_sf)
    assert got.data_ptr() == out.data_ptr() and got_sf.data_ptr() == out_sf.data_ptr()
    assert torch.equal(got.view(torch.uint8), ref.view(torch.uint8))
    assert torch.equal(got_sf, ref_sf)
    oq, osf = oracle.quant_group_wise(x.cpu(), mode, use_swizzle=use_swizzle)
    _assert_equal(got.view(torch.uint8).cpu().numpy(), oq, "codes")
    _assert_equal(got_sf.cpu().numpy(), osf, "scales")


def test_full_size_operand_properties(hq):
    """Benchmark-sized operand (8192 x 8192): checked through properties that do
    not need the whole oracle - a sampled row block is bit-exact, every scale
    byte is the smallest power of two that keeps the group inside +-448 (or one
    more for the 1.75-mantissa quirk), and dequantisation stays within the
    e4m3 half-ulp of the input."""
    m = k = 8192
    g = torch.Generator(device="cuda").manual_seed(2027)
    x = (torch.randn([m, k], generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    q, sf = hq.group_wise_quant(x)
    torch.cuda.synchronize()
    rows = torch.arange(0, m, 61)[:128]
    oq, osf = oracle.quant_group_wise(x[rows].cpu(), "w8a8-mxfp8", use_swizzle=False)
    _assert_equal(q[rows].view(torch.uint8).cpu().numpy(), oq, "sampled rows")
    sf_log = torch.from_numpy(oracle.unswizzle_sf(sf.cpu().numpy(), m))
    _assert_equal(sf_log[rows].numpy(), osf, "sampled rows scales")
    scale = torch.exp2(sf_log.float() - 127).cuda().repeat_interleave(32, dim=1)
    deq = q.float() * scale
    amax = x.float().abs().reshape(m, k // 32, 32).amax(-1)
    s = scale.reshape(m, k // 32, 32)[:, :, 0]
    assert (amax <= 448 * s).all(), "a group overflows its scale"
    assert (amax > 448 * s / 4).all(), "a scale is more than one step too large"
    err = (deq - x.float()).abs()
    assert (err <= x.float().abs() * 2 ** -4 + scale * 2 ** -10).all()
