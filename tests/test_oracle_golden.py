"""Pins the CPU oracle to fixtures produced by the reference's own CPU models
(see tests/golden/make_golden.py).  Runs without a GPU."""

import os

import numpy as np
import pytest
import torch

import oracle
from oracle.quant import ue8m0_from_scale, ue8m0_from_scale_closed_form

MODES = ("w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4")


def _bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("mode", MODES)
def test_quant_matches_reference_model(golden_dir, mode):
    d = np.load(os.path.join(golden_dir, f"quant_{mode}.npz"))
    x = _bf16(d["x_bits"])
    q, sf = oracle.quant_group_wise(x, mode, use_swizzle=True)
    assert np.array_equal(q, d["q"])
    assert np.array_equal(sf, d["sf_swizzled"])
    q2, sf2 = oracle.quant_group_wise(x, mode, use_swizzle=False)
    assert np.array_equal(q2, d["q"])
    assert np.array_equal(sf2, d["sf_logical"])


@pytest.mark.parametrize(
    "mode, key, g, floor",
    [
        # the reference's MXFP8 model clips amax at 1e-4, its FP4 models at 1e-12;
        # the kernel (and the oracle) floor at 1e-10, so compare above the clips
        ("w8a8-mxfp8", "sf_mxfp8", 32, 1e-4),
        ("w4a4-nvfp4", "sf_nvfp4", 16, 1e-10),
        ("w4a4-mxfp4", "sf_mxfp4", 32, 1e-10),
    ],
)
def test_scale_byte_for_every_bf16_amax(golden_dir, mode, key, g, floor):
    d = np.load(os.path.join(golden_dir, "amax_sweep.npz"))
    amax = _bf16(d["amax_bits"])
    x = torch.zeros([amax.numel(), g], dtype=torch.bfloat16)
    x[:, 0] = amax
    _, sf = oracle.quant_group_wise(x, mode, use_swizzle=False)
    ok = amax.float().numpy() >= floor
    assert ok.sum() > 18000
    assert np.array_equal(sf.reshape(-1)[ok], d[key][ok])


def test_all_zero_group_takes_the_kernel_floor():
    # amax floor 1e-10 -> ceil(log2(1e-10 / 448)) + 127 = 85 ; codes are zero
    x = torch.zeros([1, 32], dtype=torch.bfloat16)
    q, sf = oracle.quant_group_wise(x, "w8a8-mxfp8", use_swizzle=False)
    assert sf[0, 0] == 85 and not q.any()
    q, sf = oracle.quant_group_wise(x[:, :16], "w4a4-nvfp4", use_swizzle=False)
    assert sf[0, 0] == 1 and not q.any()


@pytest.mark.parametrize("div", [448.0, 6.0])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_closed_form_scale_equals_log2_model(div, dtype):
    """The bit-field formula the CUDA kernel uses equals the reference's
    log2-based model for every possible 16-bit amax."""
    top = 0x7F80 if dtype == torch.bfloat16 else 0x7C00
    bits = np.arange(1, top, dtype=np.uint16)
    a = torch.from_numpy(bits.view(np.int16)).view(dtype).float().numpy()
    a = np.maximum(a, np.float32(1e-10))
    s = (a / np.float32(div)).astype(np.float32)
    assert np.array_equal(ue8m0_from_scale(s), ue8m0_from_scale_closed_form(s))


def test_e4m3_encoder_matches_torch_cast():
    g = torch.Generator().manual_seed(7)
    x = torch.randn([1 << 16], generator=g) * torch.logspace(-4, 2.6, 1 << 16)
    x = x.clamp(-448, 448)
    mine = oracle.encode_e4m3_rn_satfinite(x.numpy())
    theirs = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, theirs)
    # every code decodes and re-encodes to itself (NaN patterns excluded)
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    assert np.array_equal(oracle.encode_e4m3_rn_satfinite(oracle.decode_e4m3(codes)), codes)


def test_swizzle_roundtrip_and_formula():
    rng = np.random.default_rng(3)
    sf = rng.integers(0, 255, size=(300, 24), dtype=np.uint8)
    sw = oracle.swizzle_sf(sf)
    assert sw.shape == (384, 24)
    assert np.array_equal(oracle.unswizzle_sf(sw, 300), sf)
    # padding rows are zero
    full = oracle.unswizzle_sf(sw, 384)
    assert not full[300:].any()
    # spot-check the offset formula
    off = oracle.sf_atom_offsets(384, 24)
    r, kb = 200, 13
    expect = ((r // 128) * 6 + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    assert off[r, kb] == expect
    assert sorted(off.ravel().tolist()) == list(range(384 * 24))


@pytest.mark.parametrize("mode", MODES)
def test_gemm_oracle_matches_reference_model(golden_dir, mode):
    d = np.load(os.path.join(golden_dir, f"gemm_{mode}.npz"))
    out = oracle.dense_gemm_ref(d["x"], d["w"], d["sfa"], d["sfb"], mode)
    assert torch.equal(out, _bf16(d["out_bits"]))


def test_quant_edge_cases():
    with pytest.raises(ValueError, match="Unsupported quantization mode"):
        oracle.quant_group_wise(torch.zeros([4, 64], dtype=torch.bfloat16), "w4a4-fp6")
    with pytest.raises(ValueError, match="kb_dim must be divisible by 4"):
        oracle.quant_group_wise(torch.zeros([4, 96], dtype=torch.bfloat16), "w8a8-mxfp8")
    q, sf = oracle.quant_group_wise(torch.zeros([0, 1024], dtype=torch.bfloat16), "w8a8-mxfp8")
    assert q.shape == (0, 1024) and sf.shape == (0, 32)
    # NaN -> -448, +-inf -> NaN (inf * 0) -> -448, finite next to inf -> 0
    x = torch.tensor([[float("nan")] + [1.0] * 31, [float("inf")] + [2.0] * 31], dtype=torch.bfloat16)
    q, sf = oracle.quant_group_wise(x, "w8a8-mxfp8", use_swizzle=False)
    assert q[0, 0] == 0xFE and q[1, 0] == 0xFE and sf[1, 0] == 254 and q[1, 1] == 0


def test_torch_cpu_path_equals_numpy_oracle(golden_dir):
    """The multi-threaded torch port timed by the benchmark produces the same
    bytes as the numpy oracle (and so as the reference model)."""
    from oracle.cpu_path import gemm_mxfp8_torch, quant_mxfp8_torch

    d = np.load(os.path.join(golden_dir, "quant_w8a8-mxfp8.npz"))
    x = _bf16(d["x_bits"])
    q, sf = quant_mxfp8_torch(x)
    assert np.array_equal(q.view(torch.uint8).numpy(), d["q"])
    assert np.array_equal(sf.numpy(), d["sf_logical"])
    g = torch.Generator().manual_seed(5)
    a = torch.randn([64, 256], generator=g).to(torch.bfloat16)
    b = torch.randn([96, 256], generator=g).to(torch.bfloat16)
    aq, sfa = quant_mxfp8_torch(a)
    bq, sfb = quant_mxfp8_torch(b)
    want = oracle.dense_gemm_ref(aq, bq, sfa.numpy(), sfb.numpy(), "w8a8-mxfp8", swizzled=False)
    assert torch.equal(gemm_mxfp8_torch(aq, sfa, bq, sfb), want)


def _grouped_fixture(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name))
    alpha = torch.from_numpy(d["alpha"]) if "alpha" in d else None
    bias = _bf16(d["bias_bits"]) if "bias_bits" in d else None
    return d, alpha, bias, _bf16(d["out_bits"]).float()


def _close_to_model(got, ref, bias):
    """The oracle repeats the model's arithmetic exactly, with a bias too: the product is
    rounded to bfloat16 and the bias added to that in bfloat16."""
    del bias
    assert torch.equal(got, ref)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4"])
def test_batch_oracle_matches_reference_model(golden_dir, mode):
    d, alpha, bias, ref = _grouped_fixture(golden_dir, f"batch_{mode}.npz")  # ref: [B, M, N]
    got = oracle.batch_gemm_ref(d["x"], d["w"], d["sfa"], d["sfb"], mode, alpha=alpha, bias=bias).float()
    batches, m, n = ref.shape
    for b in range(batches):
        _close_to_model(got[:, b * n:(b + 1) * n], ref[b], bias)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a8-mxfp4"])
def test_masked_oracle_matches_reference_model(golden_dir, mode):
    d, alpha, bias, ref = _grouped_fixture(golden_dir, f"masked_{mode}.npz")
    masked = d["masked_m"]
    max_m = ref.shape[0] // masked.size
    ids = np.full(ref.shape[0], -1)
    for e, cnt in enumerate(masked):
        ids[e * max_m:e * max_m + cnt] = e
    got = oracle.group_gemm_ref(d["x"], d["w"], d["sfa"], d["sfb"], ids, mode, alpha=alpha, bias=bias).float()
    # the alpha of this fixture is a power of two per expert, so it commutes with the rounding
    _close_to_model(got, ref, bias)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4", "w4a4-mxfp4", "w4a8-mxfp4"])
def test_contiguous_oracle_matches_reference_model(golden_dir, mode):
    d, alpha, bias, ref = _grouped_fixture(golden_dir, f"contiguous_{mode}.npz")
    got = oracle.group_gemm_ref(d["x"], d["w"], d["sfa"], d["sfb"], d["expert_ids"], mode, alpha=alpha,
                                bias=bias).float()
    _close_to_model(got, ref, bias)


def test_rms_norm_oracle_matches_reference_model(golden_dir):
    """The reference's fp32 RMSNorm rounded to bf16 on its own inputs
    (tests/test_rms_norm_quant.py:38-48); the quantizer applied to it is pinned above."""
    d = np.load(os.path.join(golden_dir, "rms_norm.npz"))
    got = oracle.rms_norm_ref(_bf16(d["x_bits"]), _bf16(d["w_bits"]), float(d["eps"]))
    assert torch.equal(got, _bf16(d["y_bits"]))


def test_plain_scale_dequantize_matches_reference_model(golden_dir):
    """Dequantise-then-matmul with plain row-major scales, the model of the reference's
    low-latency GEMM test (tests/test_low_latency_mma_gemm.py:62-75)."""
    d = np.load(os.path.join(golden_dir, "low_latency_w8a8-mxfp8.npz"))
    a = oracle.dequantize(d["x"], d["sfa"], "w8a8-mxfp8", swizzled=False)
    b = oracle.dequantize(d["w"], d["sfb"], "w8a8-mxfp8", swizzled=False)
    assert torch.equal(a @ b.T, torch.from_numpy(d["out"]))
