from .batch_gemm import batch_gemm
from .dense_gemm import EpilogueOp, dense_gemm, interleave_gate_up
from .group_gemm import group_contiguous_gemm, group_masked_gemm
from .group_wise_quant import group_wise_quant
from .low_latency_mma_gemm import low_latency_mma_gemm
from .rms_norm_quant import rms_norm_quant

__all__ = ["EpilogueOp", "batch_gemm", "dense_gemm", "group_contiguous_gemm", "group_masked_gemm", "group_wise_quant", "interleave_gate_up", "low_latency_mma_gemm", "rms_norm_quant"]
