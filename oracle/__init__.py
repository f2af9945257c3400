"""CPU oracle for the block-scaled quantize -> dense GEMM path.

TEST INFRASTRUCTURE ONLY.  Nothing in the ``halops_b200`` package may import
this module: it exists so that the tests, the smoke check and the CPU-baseline
leg of the benchmark can compare the CUDA path against an independent CPU
restatement of the reference's arithmetic.

Parity status: pinned.  ``tests/test_oracle_golden.py`` checks every function
here against fixtures produced by importing and running the reference's own CPU
models (``tests/test_group_wise_quant.py``, ``tests/test_dense_gemm.py`` and
``tests/utils/*.py`` of the reference); the generating script is
``tests/golden/make_golden.py``.
"""

from .quant import (  # noqa: F401
    E2M1_VALUES,
    GROUP_SIZE,
    decode_e2m1_packed,
    decode_e4m3,
    decode_ue4m3,
    decode_ue8m0,
    encode_e4m3_rn_satfinite,
    quant_group_wise,
    rms_norm_ref,
    sf_atom_offsets,
    sf_rows,
    swizzle_sf,
    ue8m0_from_scale,
    unswizzle_sf,
)
from .gemm import batch_gemm_ref, dense_gemm_ref, dequantize, group_gemm_ref  # noqa: F401
