"""The GEMM whose epilogue also gathers, ``hq_dense_gemm_allgather``, on ONE GPU.

The entry point takes one output matrix per rank.  On a single GPU the "peers'" matrices are
further buffers of the same device, so the stores that would cross NVLink land in local
memory and can be compared bit for bit with the ordinary dense GEMM: every matrix must hold
this rank's columns and nothing else may have been touched.  The multi-GPU run of the same
entry point is part of tests/test_dist_gpu.py.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _fused(aq, bq, sfa, sfb, outs, rank, sm_count=-1):
    from halops_b200 import _native

    m, k = aq.shape
    addresses = (ctypes.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
    _native.call("hq_dense_gemm_allgather", aq.data_ptr(), bq.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), addresses,
                 len(outs), rank, m, bq.shape[0], k, sfa.numel(), sfb.numel(), outs[0].stride(0), sm_count, 0,
                 aq.device.index, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("m,n_local,k,world,rank", [(256, 256, 128, 1, 0), (300, 512, 1024, 2, 1), (1000, 768, 512, 4, 2),
                                                    (2048, 1024, 2048, 8, 7), (129, 256, 256, 8, 0),
                                                    (4096, 7168, 1024, 3, 0)])
def test_every_rank_gets_this_ranks_columns(hq, m, n_local, k, world, rank):
    g = torch.Generator().manual_seed(m + world)
    a = torch.randn([m, k], generator=g).to(torch.bfloat16).cuda()
    b = (torch.randn([n_local, k], generator=g) * 0.05).to(torch.bfloat16).cuda()
    aq, sfa = hq.group_wise_quant(a)
    bq, sfb = hq.group_wise_quant(b)
    want = torch.empty([m, n_local], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, want, None, None, -1, "w8a8-mxfp8")
    for sm_count in (-1, 20):
        outs = [torch.full([m, world * n_local], 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        _fused(aq, bq, sfa, sfb, outs, rank, sm_count)
        torch.cuda.synchronize()
        assert hq.device_status() == 0
        lo, hi = rank * n_local, (rank + 1) * n_local
        for r, out in enumerate(outs):
            assert torch.equal(out[:, lo:hi], want), f"matrix {r}: columns of rank {rank} differ"
            assert bool((out[:, :lo] == 7.0).all()) and bool((out[:, hi:] == 7.0).all()), \
                f"matrix {r}: columns of another rank were written"
