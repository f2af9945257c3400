"""CPU-only checks of the drop-in boundary: the C-ABI library builds, loads and
exports every symbol the header declares, and the host-side validation raises
the reference's error texts before anything touches a device."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def native():
    from halops_b200 import build

    build.build()
    from halops_b200 import _native

    _native.lib()
    return _native


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "halops_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hq_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(native):
    names = _declared_functions()
    assert "hq_group_wise_quant" in names and "hq_dense_gemm" in names
    handle = ctypes.CDLL(native.lib_path())
    for name in names:
        assert getattr(handle, name) is not None
    assert sorted(native.SIGNATURES) == names, "ctypes table and header disagree"
    assert b"sm_100a" in native.lib().hq_version()


def test_no_torch_types_in_the_header():
    text = open(os.path.join(ROOT, "include", "halops_b200.h")).read()
    assert "torch" not in text.replace("TORCH_CHECK", "") and "at::" not in text


def test_mode_helpers(native):
    lib = native.lib()
    assert lib.hq_parse_mode(b"w8a8-mxfp8") == 0
    assert lib.hq_parse_mode(b"w4a4-mxfp4") == 1
    assert lib.hq_parse_mode(b"w4a4-nvfp4") == 2
    assert lib.hq_parse_mode(b"nvfp4") == -1
    assert [lib.hq_group_size(i) for i in range(4)] == [32, 32, 16, 0]
    assert [lib.hq_sf_rows(m) for m in (0, 1, 128, 129, 1000)] == [0, 128, 128, 256, 1024]


def _gemm_rc(native, m, n, k, mode, alpha=None, epilogue=0):
    err = ctypes.create_string_buffer(512)
    rc = native.lib().hq_dense_gemm(None, None, None, None, None, None, alpha, m, n, k, 1 << 40, 1 << 40, n,
                                    mode, epilogue, -1, 0, 0, None, err, len(err))
    return rc, err.value.decode()


@pytest.mark.parametrize("mode, m, n, k, text", [
    (0, 128, 256, 96, "No dense w8a8-mxfp8 tile for M=128 (grid M=128), N=256, K=96"),
    (0, 128, 255, 128, "No dense w8a8-mxfp8 tile for M=128 (grid M=128), N=255, K=128"),
    (2, 128, 256, 48, "No dense w4a4-nvfp4 tile for M=128 (grid M=128), N=256, K=48"),
    (0, 200, 100, 128, "No dense w8a8-mxfp8 tile for M=256 (grid M=256), N=100, K=128"),
])
def test_shape_legality_messages(native, mode, m, n, k, text):
    """Texts pinned by the reference's tests/test_dense_gemm.py:398-492."""
    alpha = ctypes.cast(16, ctypes.c_void_p) if mode == 2 else None
    rc, msg = _gemm_rc(native, m, n, k, mode, alpha)
    assert rc == 1 and text in msg


def test_gemm_argument_rules(native):
    rc, msg = _gemm_rc(native, 128, 256, 512, 1, alpha=ctypes.cast(16, ctypes.c_void_p))
    assert rc == 1 and "does not take alpha" in msg
    rc, msg = _gemm_rc(native, 128, 256, 512, 2, alpha=None)
    assert rc == 1 and "requires alpha" in msg
    rc, msg = _gemm_rc(native, 128, 256, 512, 0, epilogue=4)
    assert rc == 3 and "Unsupported epilogue" in msg
    rc, msg = _gemm_rc(native, 128, 256, 512, 7)
    assert rc == 1 and "Unsupported mode" in msg
    assert _gemm_rc(native, 0, 256, 512, 0)[0] == 0  # empty problem: nothing to do


def test_quant_argument_rules(native):
    err = ctypes.create_string_buffer(512)
    f = native.lib().hq_group_wise_quant
    assert f(None, 96, 0, 128, 96, 0, 1, 0, None, None, 0, None, err, len(err)) == 1
    assert b"scale kb_dim must be divisible by 4" in err.value
    assert f(None, 100, 0, 128, 100, 0, 0, 0, None, None, 0, None, err, len(err)) == 1
    assert b"k must be divisible by the quantization group size (32)" in err.value
    assert f(None, 1024, 0, 128, 1024, 9, 1, 0, None, None, 0, None, err, len(err)) == 1
    assert b"Unsupported quantization mode" in err.value
    assert f(None, 1024, 5, 128, 1024, 0, 1, 0, None, None, 0, None, err, len(err)) == 1
    assert b"bfloat16 or float16" in err.value
    assert f(None, 1024, 0, 0, 1024, 0, 1, 0, None, None, 0, None, err, len(err)) == 0  # m = 0


def test_python_wrapper_errors_without_a_device():
    import halops_b200 as hq

    x = torch.zeros([128, 1024], dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match=re.escape("Unsupported quantization mode")):
        hq.group_wise_quant(x, mode="w4a4-fp6")
    with pytest.raises(RuntimeError, match=re.escape("scale kb_dim must be divisible by 4")):
        hq.group_wise_quant(torch.zeros([128, 96], dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="no CPU path"):
        hq.group_wise_quant(x)

    def empties(m, n, k, mode, x_shape=None, out_shape=None):
        if mode == "w8a8-mxfp8":
            a = torch.empty(x_shape or [m, k], dtype=torch.float8_e4m3fn)
            w = torch.empty([n, k], dtype=torch.float8_e4m3fn)
            sfa, sfb = torch.empty([m, k // 32], dtype=torch.uint8), torch.empty([n, k // 32], dtype=torch.uint8)
            alpha = None
        else:
            a = torch.empty(x_shape or [m, k // 2], dtype=torch.uint8)
            w = torch.empty([n, k // 2], dtype=torch.uint8)
            g = 16 if mode == "w4a4-nvfp4" else 32
            sfa, sfb = torch.empty([m, k // g], dtype=torch.uint8), torch.empty([n, k // g], dtype=torch.uint8)
            alpha = torch.ones([1]) if mode == "w4a4-nvfp4" else None
        return a, w, sfa, sfb, torch.empty(out_shape or [m, n], dtype=torch.bfloat16), alpha

    cases = [
        ("w8a8-mxfp8", 128, 256, 96, None, None, "No dense w8a8-mxfp8 tile for M=128 (grid M=128), N=256, K=96"),
        ("w8a8-mxfp8", 128, 255, 128, None, None, "No dense w8a8-mxfp8 tile for M=128 (grid M=128), N=255, K=128"),
        ("w4a4-nvfp4", 128, 256, 48, None, None, "No dense w4a4-nvfp4 tile for M=128 (grid M=128), N=256, K=48"),
        ("w8a8-mxfp8", 128, 256, 128, [128, 1, 128], None, "input must be a 2D tensor"),
        ("w8a8-mxfp8", 128, 256, 128, None, [128, 256, 1], "output must be a 2D tensor"),
    ]
    for mode, m, n, k, xs, os_, text in cases:
        a, w, sfa, sfb, out, alpha = empties(m, n, k, mode, xs, os_)
        with pytest.raises(RuntimeError, match=re.escape(text)):
            hq.dense_gemm(a, w, sfa, sfb, out, None, alpha, -1, mode)

    a, w, sfa, sfb, out, _ = empties(128, 256, 512, "w4a4-mxfp4")
    with pytest.raises(RuntimeError, match=re.escape("does not take alpha")):
        hq.dense_gemm(a, w, sfa, sfb, out, None, torch.ones([1]), -1, "w4a4-mxfp4")
    a, w, _, _, out, _ = empties(128, 256, 512, "w4a4-mxfp4")
    bad = torch.empty([128, 32], dtype=torch.uint8), torch.empty([256, 32], dtype=torch.uint8)
    with pytest.raises(RuntimeError, match=re.escape("scale-factor shape does not match mode")):
        hq.dense_gemm(a, w, bad[0], bad[1], out, None, None, -1, "w4a4-mxfp4")
    a, w, sfa, sfb, out, _ = empties(200, 1024, 1024, "w8a8-mxfp8")
    with pytest.raises(RuntimeError, match=re.escape("multiple of 256")):
        hq.dense_gemm(a, w, torch.empty([256, 32], dtype=torch.uint8), sfb, out, torch.zeros([1024], dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="Unsupported mode"):
        hq.dense_gemm(a, w, sfa, sfb, out, mode="nvfp4")
    with pytest.raises(RuntimeError, match="no CPU path"):
        a, w, sfa, sfb, out, _ = empties(128, 256, 512, "w8a8-mxfp8")
        hq.dense_gemm(a, w, sfa, sfb, out)


def test_batch_gemm_rules_without_a_device(native):
    """Host checks of the batch GEMM (texts of the reference's tests/test_batch_gemm.py:313-363,
    537-590) through the C entry point with null operands and through the Python wrapper."""
    import halops_b200 as hq

    def rc(batches, m, n, k, mode, alpha=None, bias=None, epilogue=0):
        err = ctypes.create_string_buffer(512)
        code = native.lib().hq_batch_gemm(None, None, None, None, None, bias, alpha, batches, m, n, k, 1 << 40,
                                          1 << 40, batches * n, mode, epilogue, -1, 0, 0, None, err, len(err))
        return code, err.value.decode()

    fake = ctypes.cast(16, ctypes.c_void_p)
    code, msg = rc(2, 128, 256, 96, 0)
    assert code == 1 and "No batch w8a8-mxfp8 tile for M=128 (grid M=256), N=256, K=96" in msg
    code, msg = rc(2, 128, 256, 256, 2)
    assert code == 1 and "requires alpha input (per-batch scaling)" in msg
    code, msg = rc(2, 128, 256, 512, 1, alpha=fake)
    assert code == 1 and "does not take alpha; the per-batch scaling factor" in msg
    code, msg = rc(2, 128, 256, 256, 2, alpha=fake, bias=fake)
    assert code == 1 and "W4A4 batch GEMM does not support bias" in msg
    code, msg = rc(2, 128, 256, 128, 0, epilogue=1)
    assert code == 3 and "Unsupported epilogue 1" in msg
    assert rc(0, 128, 256, 128, 0)[0] == 0 and rc(2, 0, 256, 128, 0)[0] == 0
    err = ctypes.create_string_buffer(512)
    assert native.lib().hq_batch_gemm(fake, fake, fake, fake, fake, None, None, 2, 100, 256, 128, 256 * 4 - 1,
                                      1 << 40, 512, 0, 0, -1, 0, 0, None, err, len(err)) == 1
    assert b"sfa must hold whole 128-row SfAtoms over the stacked rows" in err.value

    x = torch.empty([2, 128, 128], dtype=torch.float8_e4m3fn)
    w = torch.empty([2, 256, 128], dtype=torch.float8_e4m3fn)
    sfa = torch.empty([256, 4], dtype=torch.uint8)
    sfb = torch.empty([2, 256, 4], dtype=torch.uint8)
    out = torch.empty([128, 512], dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="input must be a 3D tensor"):
        hq.batch_gemm(x[0], w, sfa, sfb, out)
    with pytest.raises(RuntimeError, match="weight batch dim must match input batch dim, got 3"):
        hq.batch_gemm(x, torch.empty([3, 256, 128], dtype=torch.float8_e4m3fn), sfa, sfb, out)
    with pytest.raises(RuntimeError, match=re.escape("output must be a 2D tensor of shape [M, B * N]")):
        hq.batch_gemm(x, w, sfa, sfb, out.view(2, 64, 512))
    with pytest.raises(RuntimeError, match=re.escape("output shape must be [M, B * N]")):
        hq.batch_gemm(x, w, sfa, sfb, out[:, :256])
    with pytest.raises(RuntimeError, match="Unsupported mode: w2a2"):
        hq.batch_gemm(x, w, sfa, sfb, out, mode="w2a2")
    with pytest.raises(RuntimeError, match="no CPU path"):
        hq.batch_gemm(x, w, sfa, sfb, out)
    assert "mode=batch" in hq.describe_group_tile("batch", 4, 200, 256, 128)


def test_group_gemm_rules_without_a_device(native):
    """Host checks of the masked / contiguous grouped GEMMs (texts of the reference's
    tests/test_group_masked_gemm.py:840-866 and tests/test_group_contiguous_gemm.py:628-652)."""
    import halops_b200 as hq

    fake = ctypes.cast(16, ctypes.c_void_p)
    err = ctypes.create_string_buffer(512)
    masked = native.lib().hq_group_masked_gemm
    contiguous = native.lib().hq_group_contiguous_gemm
    big = 1 << 40
    assert masked(None, None, None, None, None, None, None, None, 2, 129, 256, 128, big, big, 256, 0, -1, 1, 0, None,
                  err, len(err)) == 1
    assert b"No masked w8a8-mxfp8 tile for M=129 (grid M=258), N=256, K=128" in err.value
    assert masked(None, None, None, None, None, None, None, None, 2, 0, 256, 128, big, big, 256, 0, -1, 1, 0, None,
                  err, len(err)) == 1
    assert b"max_m_per_expert must be greater than 0, got 0" in err.value
    assert masked(None, None, None, None, None, None, fake, fake, 2, 128, 128, 512, big, big, 128, 2, -1, 1, 0, None,
                  err, len(err)) == 1
    assert b"W4A4 mode does not support bias yet." in err.value
    assert masked(None, None, None, None, None, None, None, None, 2, 128, 128, 512, big, big, 128, 2, -1, 1, 0, None,
                  err, len(err)) == 1
    assert b"requires alpha input (per-expert scaling factor)" in err.value
    assert contiguous(None, None, None, None, None, None, None, None, 1, 129, 256, 128, big, big, 256, 0, -1, 1, 0,
                      None, err, len(err)) == 1
    assert b"No contiguous w8a8-mxfp8 tile for M=129 (grid M=129), N=256, K=128" in err.value
    assert contiguous(None, None, None, None, None, None, None, fake, 1, 128, 256, 512, big, big, 256, 1, -1, 1, 0,
                      None, err, len(err)) == 1
    assert b"does not take alpha; the per-expert scaling factor" in err.value
    assert contiguous(None, None, None, None, None, None, None, None, 1, 0, 256, 128, big, big, 256, 0, -1, 1, 0,
                      None, err, len(err)) == 0  # no rows: nothing to do
    # mode 3: e4m3 activations x packed e2m1 weights (tests/test_group_masked_gemm.py:727-768)
    assert masked(None, None, None, None, None, None, fake, None, 2, 128, 128, 512, big, big, 128, 3, -1, 1, 0, None,
                  err, len(err)) == 1
    assert b"W4A8 mode does not support bias yet." in err.value
    assert contiguous(None, None, None, None, None, None, None, fake, 1, 128, 256, 512, big, big, 256, 3, -1, 1, 0,
                      None, err, len(err)) == 1
    assert b"W4A8 mode does not take alpha" in err.value

    x = torch.empty([256, 128], dtype=torch.float8_e4m3fn)
    w = torch.empty([2, 256, 128], dtype=torch.float8_e4m3fn)
    sfa = torch.empty([256, 4], dtype=torch.uint8)
    sfb = torch.empty([2, 256, 4], dtype=torch.uint8)
    out = torch.empty([256, 256], dtype=torch.bfloat16)
    counts = torch.full([2], 128, dtype=torch.int32)
    ids = torch.zeros([256], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="masked_m must have dtype torch.int32"):
        hq.group_masked_gemm(x, w, sfa, sfb, counts.long(), out, None, None, 128)
    with pytest.raises(RuntimeError, match=re.escape("masked_m shape must be [num_experts], got 1, expected 2")):
        hq.group_masked_gemm(x, w, sfa, sfb, counts[:1], out, None, None, 128)
    with pytest.raises(RuntimeError, match="input M must equal num_experts . max_m_per_expert, got 256, expected 128"):
        hq.group_masked_gemm(x, w, sfa, sfb, counts, out, None, None, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        hq.group_masked_gemm(x, w, sfa, sfb, counts, out, None, None, 128)
    with pytest.raises(RuntimeError, match="expert_ids must have dtype torch.int32"):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids.long(), out)
    with pytest.raises(RuntimeError, match=re.escape("output shape must be [M, N], got [256, 128], expected [256, 256]")):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids, out[:, :128])
    with pytest.raises(RuntimeError, match="no CPU path"):
        hq.group_contiguous_gemm(x, w, sfa, sfb, ids, out)
    assert "mode=masked" in hq.describe_group_tile("masked", 20, 64, 7168, 3584)
    assert "mode=contiguous" in hq.describe_group_tile("contiguous", 16, 256, 7168, 3584)
    assert "w4a8-mxfp4" in hq.describe_group_tile("masked", 8, 128, 7168, 2048, "w4a8-mxfp4", sm_count=148)
    with pytest.raises(RuntimeError):
        hq.describe_group_tile("batch", 8, 128, 7168, 2048, "w4a8-mxfp4", sm_count=148)


def test_low_latency_rules_without_a_device(native):
    """Host checks of the plain-scale M <= 16 GEMM (texts of the reference's
    tests/test_low_latency_mma_gemm.py:297-345)."""
    import halops_b200 as hq

    fake = ctypes.cast(16, ctypes.c_void_p)
    f = native.lib().hq_low_latency_gemm

    def rc(m, n, n2, k1, k2, strides=(128, 128, 128, 128), a2=None, b2=None, sfa2=None, sfb2=None, out2=None,
           sigmoid=0):
        err = ctypes.create_string_buffer(512)
        code = f(None, None, None, None, None, a2, b2, sfa2, sfb2, out2, m, n, n2, k1, k2, *strides, n, n2, sigmoid,
                 -1, 1, 0, None, err, len(err))
        return code, err.value.decode()

    assert "supports M <= 16, got M=17" in rc(17, 512, 0, 4096, 0)[1]
    assert "weight rows must be divisible by 8, got 516 and 0" in rc(8, 516, 0, 256, 0, strides=(16, 16, 0, 0))[1]
    assert "K must be divisible by 256, got K=1152" in rc(8, 512, 0, 1152, 0, strides=(48, 48, 0, 0))[1]
    assert "plain row-major" in rc(8, 512, 0, 1024, 0, strides=(36, 32, 0, 0))[1]
    assert "weight2 / sfb2 must come with" in rc(8, 512, 0, 2048, 0, b2=fake, sfb2=fake)[1]
    assert "does not support input2 or output2" in rc(8, 512, 512, 2048, 0, b2=fake, sfb2=fake, out2=fake, sigmoid=1)[1]
    assert "K1 must be a multiple of 512, got K1=1920" in rc(8, 512, 0, 1920, 2176, a2=fake, b2=fake, sfa2=fake,
                                                             sfb2=fake)[1]
    assert rc(0, 512, 0, 1024, 0, strides=(32, 32, 0, 0))[0] == 0  # no rows: nothing to do

    x = torch.empty([8, 1024], dtype=torch.float8_e4m3fn)
    w = torch.empty([512, 1024], dtype=torch.float8_e4m3fn)
    sfa, sfb = torch.empty([8, 32], dtype=torch.uint8), torch.empty([512, 32], dtype=torch.uint8)
    out = torch.empty([8, 512], dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="plain row-major"):
        hq.low_latency_mma_gemm(x, w, torch.empty([128, 32], dtype=torch.uint8), sfb, out)
    with pytest.raises(RuntimeError, match="supports M <= 16"):
        hq.low_latency_mma_gemm(torch.empty([17, 1024], dtype=torch.float8_e4m3fn), w, sfa, sfb, out)
    with pytest.raises(RuntimeError, match="no CPU path"):
        hq.low_latency_mma_gemm(x, w, sfa, sfb, out)


def test_enum_and_interleave():
    import halops_b200 as hq

    assert [int(e) for e in hq.EpilogueOp] == [0, 1, 2, 3, 4, 5]
    assert hq.EpilogueOp.SituQuant == 4
    t = torch.arange(64).reshape(64, 1)
    r = hq.interleave_gate_up(t).reshape(-1)
    assert r[:16].tolist() == list(range(16)) and r[16:32].tolist() == list(range(32, 48))
    assert r[32:48].tolist() == list(range(16, 32))


def test_decode_unit_deal_is_consistent(native):
    """The small-M kernel's deal of (128 weight rows x 256 bytes of K) units to the CTAs: every
    unit once, contiguous runs, distinct scratch slots per tile -- checked by the library's
    host-side self-check over many shapes and SM counts, with and without the even split."""
    from halops_b200 import _native

    for n in list(range(64, 2049, 64)) + [4736, 7168, 8192, 24576, 32768, 57344]:
        for k in (128, 256, 384, 1024, 1152, 1536, 2048, 4096, 8192):
            for sm in (1, 2, 7, 74, 132, 148, 160):
                for force_split in (0, 1, 2):
                    _native.call("hq_selftest_decode_plan", n, k, sm, force_split)
    with pytest.raises(RuntimeError, match="multiple of 128"):
        _native.call("hq_selftest_decode_plan", 128, 100, 148, 0)


def test_describe_tile(native):
    import halops_b200 as hq

    assert "256x256/128 pair=1" in hq.describe_tile(8192, 8192, 8192, sm_count=148)
    assert "128x256/256 pair=0" in hq.describe_tile(4096, 14336, 4096, "w4a4-nvfp4", sm_count=148)
    assert "256x256/128 pair=1" in hq.describe_tile(8192, 4096, 4096, sm_count=148)
    # 144 single-CTA tiles fit one wave, 80 pair tiles need two
    assert "128x256/128 pair=0" in hq.describe_tile(1152, 4096, 4096, sm_count=148)
    # small M: the operand-swapped kernel; whole tiles per CTA, or every tile dealt to several
    # CTAs when the weight has too few tiles to keep HBM busy
    assert "swap 128x16/256 pair=0 splitk=0 ctas=56" in hq.describe_tile(8, 7168, 2048, sm_count=148)
    assert "swap 128x64/256 pair=0 splitk=0 ctas=148" in hq.describe_tile(64, 24576, 1536, sm_count=148)
    assert "swap 128x16/256 pair=0 splitk=0 ctas=64" in hq.describe_tile(8, 8192, 1024, sm_count=148)
    assert "swap 128x64/256 pair=0 splitk=1 ctas=128" in hq.describe_tile(64, 4096, 8192, sm_count=148)
    assert "swap" not in hq.describe_tile(65, 7168, 2048, sm_count=148)
    with pytest.raises(RuntimeError, match="No dense"):
        hq.describe_tile(128, 96, 128, sm_count=148)


def test_product_never_imports_the_oracle():
    """The library must not route through the CPU oracle."""
    pkg = os.path.join(ROOT, "halops_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read(), f


def test_gemm_allgather_rules_without_a_device(native):
    import ctypes

    from halops_b200 import _native

    def call(world, rank, m, n_local, k, ldo):
        outs = (ctypes.c_void_p * 8)(*([256] * 8))
        _native.call("hq_dense_gemm_allgather", 256, 256, 256, 256, outs, world, rank, m, n_local, k, 1 << 40, 1 << 40,
                     ldo, -1, 0, 0, None)

    with pytest.raises(RuntimeError, match="world must be"):
        call(9, 0, 256, 256, 128, 256 * 9)
    with pytest.raises(RuntimeError, match="world must be"):
        call(2, 2, 256, 256, 128, 512)
    with pytest.raises(RuntimeError, match="multiple of 256"):
        call(2, 0, 256, 128, 128, 256)
    with pytest.raises(RuntimeError, match="multiple of 256"):
        call(2, 0, 128, 256, 128, 512)
    with pytest.raises(RuntimeError, match="row stride"):
        call(2, 0, 256, 256, 128, 256)
