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
    for name in ("group_wise_quant", "dense_gemm", "interleave_gate_up"):
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    tq, tdg, gu = _import_reference(args.reference)
    make_quant(tq, args.out)
    make_amax_sweep(tq, args.out)
    make_gemm(tdg, gu, args.out)
    for f in sorted(os.listdir(args.out)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(args.out, f)))


if __name__ == "__main__":
    main()
