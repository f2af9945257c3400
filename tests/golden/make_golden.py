"""Generate the golden fixtures in this directory from the reference's own CPU models.

Run once in a container that has the reference checkout (it is NOT needed to
run the tests; the fixtures are committed):

    python tests/golden/make_golden.py --reference /path/to/HALOps

The reference's test modules are imported as they are (pure numpy / torch CPU
code); a stub ``halops`` module stands in for the GPU extension they import at
the top but never call here.  Outputs:

* ``quant_<mode>.npz``  - seeded bf16 inputs and the reference models' quantised
  bytes, logical scales and SfAtom-swizzled scales
  (``ref_per_token_cast_to_fp8 / _nvfp4 / _mxfp4``, ``ref_reorder_sf_to_cutlass``).
* ``amax_sweep.npz``    - the scale byte the reference models assign to every
  finite non-negative bf16 amax (one group per value), all three modes.
* ``gemm_<mode>.npz``   - operands quantised by the reference's
  ``per_token_cast_* / per_block_cast_*`` helpers, swizzled with
  ``reorder_sf_to_cutlass``, and the reference ``ref_gemm`` / ``ref_gemm_w4a4``
  bf16 output.
* ``batch_<mode>.npz``, ``masked_<mode>.npz``, ``contiguous_<mode>.npz`` (also ``w4a8-mxfp4``) - inputs built
  by the input builders of the reference's ``tests/test_batch_gemm.py``,
  ``tests/test_group_masked_gemm.py`` and ``tests/test_group_contiguous_gemm.py`` and the
  outputs of their CPU models (``ref_batch_gemm_fp8 / _fp4``, ``ref_group_masked_gemm`` /
  ``_w4a4``, ``ref_group_contiguous_gemm``).
* ``rms_norm.npz``, ``low_latency_w8a8-mxfp8.npz`` - inputs and CPU models of
  ``tests/test_rms_norm_quant.py`` and ``tests/test_low_latency_mma_gemm.py``.
"""

from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root: str):
    stub = types.ModuleType("halops")
    for name in ("group_wise_quant", "dense_gemm", "interleave_gate_up", "batch_gemm", "group_masked_gemm",
                 "group_contiguous_gemm", "low_latency_mma_gemm", "rms_norm_quant"):
        setattr(stub, name, None)

    class _EpilogueOp:  # only attribute access at import time
        Identity, Quant, GateMulQuant, Sigmoid, SituQuant, SigmoidGateMulQuant = range(6)

    stub.EpilogueOp = _EpilogueOp
    sys.modules["halops"] = stub
    sys.path.insert(0, root)
    import tests.test_dense_gemm as tdg  # noqa: E402
    import tests.test_group_wise_quant as tq  # noqa: E402
    import tests.utils.gemm_utils as gu  # noqa: E402
    assert os.path.abspath(tq.__file__).startswith(os.path.abspath(root))
    return tq, tdg, gu


def _import_grouped():
    import tests.test_batch_gemm as tbg  # noqa: E402
    import tests.test_group_contiguous_gemm as tcg  # noqa: E402
    import tests.test_group_masked_gemm as tmg  # noqa: E402
    return tbg, tmg, tcg


def _bf16_bits(x: torch.Tensor) -> np.ndarray:
    return x.view(torch.int16).numpy().view(np.uint16).copy()


def _quant_inputs(seed: int, m: int, k: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn([m, k], generator=g, dtype=torch.float32)
    # rows with other magnitudes: weights-like, outliers, a constant block
    x[1] *= 0.02
    x[2] *= 37.0
    x[3, : k // 2] = 1.75  # amax/448 and amax/6 hit the power-of-two quirk or its neighbourhood
    x[4, : k // 2] = 1.5
    x[5] = x[5] / torch.sqrt(torch.randn([k], generator=g).pow(2) + 1e-3)  # heavy tails
    return x.to(torch.bfloat16)


def make_quant(tq, out_dir: str) -> None:
    m, k = 160, 512
    x = _quant_inputs(2026, m, k)
    m_sf = (m + 127) // 128 * 128
    for mode, fn, g in (
        ("w8a8-mxfp8", tq.ref_per_token_cast_to_fp8, 32),
        ("w4a4-nvfp4", tq.ref_per_token_cast_to_nvfp4, 16),
        ("w4a4-mxfp4", tq.ref_per_token_cast_to_mxfp4, 32),
    ):
        res = fn(x, g)
        q, sf = res[0], res[1]
        kb = k // g
        padded = torch.zeros([m_sf, kb], dtype=torch.uint8)
        padded[:m] = sf
        sf_sw = tq.ref_reorder_sf_to_cutlass(padded, m_sf, kb)
        np.savez_compressed(
            os.path.join(out_dir, f"quant_{mode}.npz"),
            x_bits=_bf16_bits(x),
            q=q.view(torch.uint8).numpy(),
            sf_logical=sf.numpy(),
            sf_swizzled=sf_sw.numpy(),
        )


def make_amax_sweep(tq, out_dir: str) -> None:
    bits = np.arange(0, 0x7F80, dtype=np.uint16)  # every finite non-negative bf16
    amax = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
    out = {"amax_bits": bits}
    for mode, fn, g in (
        ("mxfp8", tq.ref_per_token_cast_to_fp8, 32),
        ("nvfp4", tq.ref_per_token_cast_to_nvfp4, 16),
        ("mxfp4", tq.ref_per_token_cast_to_mxfp4, 32),
    ):
        x = torch.zeros([bits.size, g], dtype=torch.bfloat16)
        x[:, 0] = amax
        out[f"sf_{mode}"] = fn(x, g)[1].numpy().reshape(-1)
    np.savez_compressed(os.path.join(out_dir, "amax_sweep.npz"), **out)


def make_gemm(tdg, gu, out_dir: str) -> None:
    torch.manual_seed(2026)
    m, n, k = 96, 128, 256
    inp = tdg.make_w8a8_mxfp8_inputs(m, n, k)
    ref = tdg.ref_gemm(inp["x"], inp["w"], inp["sfa_logical"], inp["sfb_logical"])
    np.savez_compressed(
        os.path.join(out_dir, "gemm_w8a8-mxfp8.npz"),
        x=inp["x"].view(torch.uint8).numpy(), w=inp["w"].view(torch.uint8).numpy(),
        sfa=inp["sfa"].numpy(), sfb=inp["sfb"].numpy(), out_bits=_bf16_bits(ref),
    )
    for mode, maker in (("w4a4-nvfp4", tdg.make_nvfp4_inputs), ("w4a4-mxfp4", tdg.make_mxfp4_inputs)):
        m, n, k = 96, 128, 512
        inp = maker(m, n, k)
        ref = tdg.ref_gemm_w4a4(inp["x_fp4_float"], inp["w_fp4_float"])
        np.savez_compressed(
            os.path.join(out_dir, f"gemm_{mode}.npz"),
            x=inp["x_packed"].numpy(), w=inp["w_packed"].numpy(),
            sfa=inp["sfa"].numpy(), sfb=inp["sfb"].numpy(), out_bits=_bf16_bits(ref),
        )


def _u8(t: torch.Tensor) -> np.ndarray:
    return (t if t.dtype == torch.uint8 else t.contiguous().view(torch.uint8)).numpy()


def make_grouped(out_dir: str) -> None:
    tbg, tmg, tcg = _import_grouped()
    torch.manual_seed(2027)
    # batch, MXFP8 with bias: 100 rows per batch, so 128-row tiles straddle two batches
    inp = tbg.make_w8a8_mxfp8_inputs(3, 100, 128, 256, add_bias=True)
    ref = tbg.ref_batch_gemm_fp8(inp["input_fp8"], inp["weight_fp8"], inp["sfa_logical"], inp["sfb_logical"],
                                 bias=inp["bias"])
    np.savez_compressed(
        os.path.join(out_dir, "batch_w8a8-mxfp8.npz"), x=_u8(inp["input_fp8"]), w=_u8(inp["weight_fp8"]),
        sfa=inp["sfa"].numpy(), sfb=inp["sfb"].numpy(), bias_bits=_bf16_bits(inp["bias"]), out_bits=_bf16_bits(ref))
    inp = tbg.make_nvfp4_inputs(2, 64, 128, 512)
    ref = tbg.ref_batch_gemm_fp4(inp["x_fp4_float"], inp["w_fp4_float"])
    np.savez_compressed(
        os.path.join(out_dir, "batch_w4a4-nvfp4.npz"), x=inp["input_packed"].numpy(), w=inp["weight_packed"].numpy(),
        sfa=inp["sfa"].numpy(), sfb=inp["sfb"].numpy(), alpha=inp["alpha"].numpy(), out_bits=_bf16_bits(ref))
    # masked: partly filled, full and empty slots
    inp = tmg.make_w8a8_mxfp8_inputs(128, 3, 128, 256, full_x=False, masked_m=[17, 128, 0], add_bias=True)
    ref = tmg.ref_group_masked_gemm(inp.x, inp.w, inp.sfa_logical, inp.sfb_logical, inp.masked_m, 128, 3,
                                    bias=inp.bias)
    np.savez_compressed(
        os.path.join(out_dir, "masked_w8a8-mxfp8.npz"), x=_u8(inp.x), w=_u8(inp.w), sfa=inp.sfa.numpy(),
        sfb=inp.sfb.numpy(), masked_m=inp.masked_m.numpy(), bias_bits=_bf16_bits(inp.bias), out_bits=_bf16_bits(ref))
    inp = tmg.make_nvfp4_inputs(64, 4, 128, 512, full_x=False, masked_m=[64, 5, 0, 33], alpha=[1.0, 0.5, 2.0, 0.25])
    ref = tmg.ref_group_masked_gemm_w4a4(inp.x_fp4_float, inp.w_fp4_float, inp.masked_m, 64, 4, alpha=inp.alpha)
    np.savez_compressed(
        os.path.join(out_dir, "masked_w4a4-nvfp4.npz"), x=inp.x_packed.numpy(), w=inp.w_packed.numpy(),
        sfa=inp.sfa.numpy(), sfb=inp.sfb.numpy(), masked_m=inp.masked_m.numpy(), alpha=inp.alpha.numpy(),
        out_bits=_bf16_bits(ref))
    # contiguous: three experts with 128 rows each, per-expert bias
    inp = tcg.make_w8a8_mxfp8_inputs(384, 128, 256, 3, 64, add_bias=True)
    ref = tcg.ref_group_contiguous_gemm(inp.x, inp.w, inp.sfa_logical, inp.sfb_logical, inp.expert_ids,
                                        inp.num_experts, token_nums=inp.token_nums, bias=inp.bias)
    np.savez_compressed(
        os.path.join(out_dir, "contiguous_w8a8-mxfp8.npz"), x=_u8(inp.x), w=_u8(inp.w), sfa=inp.sfa.numpy(),
        sfb=inp.sfb.numpy(), expert_ids=inp.expert_ids.numpy(), bias_bits=_bf16_bits(inp.bias),
        out_bits=_bf16_bits(ref))
    # (after the others, so that their random streams stay as they were)
    # masked, FP8 activations x packed FP4 weights: the reference's partial case
    # (tests/test_group_masked_gemm.py:640-650) and its model for it
    inp = tmg.make_w4a8_mxfp4_inputs(128, 4, 128, 512, full_x=False, masked_m=[11, 37, 89, 128])
    ref = tmg.ref_group_masked_gemm_w4a4(inp.x_deq_float, inp.w_fp4_float, inp.masked_m, 128, 4)
    np.savez_compressed(
        os.path.join(out_dir, "masked_w4a8-mxfp4.npz"), x=_u8(inp.x), w=inp.w_packed.numpy(),
        sfa=inp.sfa.numpy(), sfb=inp.sfb.numpy(), masked_m=inp.masked_m.numpy(), out_bits=_bf16_bits(ref))
    # contiguous in the FP4 modes and the mixed one (tests/test_group_contiguous_gemm.py:223-470)
    for mode, make in (("w4a4-nvfp4", tcg.make_nvfp4_inputs), ("w4a4-mxfp4", tcg.make_mxfp4_inputs),
                       ("w4a8-mxfp4", tcg.make_w4a8_mxfp4_inputs)):
        inp = make(384, 128, 512, 3, 64)
        mixed = mode == "w4a8-mxfp4"
        ref = tcg.ref_group_contiguous_gemm_w4a4(inp.x_deq_float if mixed else inp.x_fp4_float, inp.w_fp4_float,
                                                 inp.expert_ids, inp.num_experts)
        extra = {"alpha": inp.alpha.numpy()} if mode == "w4a4-nvfp4" else {}
        np.savez_compressed(
            os.path.join(out_dir, f"contiguous_{mode}.npz"), x=_u8(inp.x) if mixed else inp.x_packed.numpy(),
            w=inp.w_packed.numpy(), sfa=inp.sfa.numpy(), sfb=inp.sfb.numpy(), expert_ids=inp.expert_ids.numpy(),
            out_bits=_bf16_bits(ref), **extra)
    # rms_norm_quant: the reference's inputs and its fp32 RMSNorm rounded to bf16
    # (tests/test_rms_norm_quant.py:38-48); the quantizer that follows is pinned above
    import tests.test_rms_norm_quant as trn  # noqa: E402
    x, w = trn.make_inputs(40, 1024)
    np.savez_compressed(os.path.join(out_dir, "rms_norm.npz"), x_bits=_bf16_bits(x), w_bits=_bf16_bits(w),
                        y_bits=_bf16_bits(trn.ref_rms_norm(x, w)), eps=np.float32(trn.EPS))
    # low_latency_mma_gemm: operands with a power of two per (row, k-group) as the reference
    # builds them (tests/test_low_latency_mma_gemm.py:31-43), quantised by its CPU recipe, plain
    # row-major scales, and its dequantise-then-matmul model (:67-75)
    import tests.test_low_latency_mma_gemm as tll  # noqa: E402
    import tests.utils.gemm_utils as gu  # noqa: E402
    aq, sfa = gu.per_token_cast_to_fp8(tll.make_bf16(5, 1280, 0.1), 32)
    bq, sfb = gu.per_token_cast_to_fp8(tll.make_bf16(136, 1280, 1280 ** -0.5), 32)
    np.savez_compressed(os.path.join(out_dir, "low_latency_w8a8-mxfp8.npz"), x=_u8(aq), w=_u8(bq), sfa=sfa.numpy(),
                        sfb=sfb.numpy(), out=tll.reference(aq, sfa, bq, sfb).numpy())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    tq, tdg, gu = _import_reference(args.reference)
    make_quant(tq, args.out)
    make_amax_sweep(tq, args.out)
    make_gemm(tdg, gu, args.out)
    make_grouped(args.out)
    for f in sorted(os.listdir(args.out)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(args.out, f)))


if __name__ == "__main__":
    main()
