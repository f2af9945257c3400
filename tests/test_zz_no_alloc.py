"""The allocation-free small-M entry point, ``hq_dense_gemm_small_m_noalloc``.

Some callers of this library cannot let it allocate device memory: code that is inside a
stream capture (a ``cudaMalloc`` there fails the capture), servers that hand the whole GPU
to their own memory pool at start-up, real-time paths that must not wait on the allocator.
``hq_dense_gemm`` takes the scratch memory of its small-M kernel from ``cudaMalloc`` the
first time a stream needs it; this entry point keeps the scratch in a fixed array inside
the library instead and so allocates nothing, at the price of limits on the problem size.

The test calls it through the C ABI, twice in a row per shape (the array keeps the previous
call's contents, so the second call starts from a used array), and compares with the
ordinary entry point on the same operands.  This file is collected last on purpose.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = dict(rtol=2e-2, atol=2e-3)  # the MXFP8 tolerance of the other GEMM tests


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def _operands(hq, m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn([m, k], generator=g).to(torch.bfloat16).cuda()
    b = (torch.randn([n, k], generator=g) * 0.02).to(torch.bfloat16).cuda()
    aq, sfa = hq.group_wise_quant(a)
    bq, sfb = hq.group_wise_quant(b)
    return aq, bq, sfa, sfb


def _noalloc(aq, bq, sfa, sfb, out, epilogue=0, sm_count=-1):
    from halops_b200 import _native

    m, k = aq.shape
    n = bq.shape[0]
    _native.call("hq_dense_gemm_small_m_noalloc", aq.data_ptr(), bq.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                 out.data_ptr(), m, n, k, sfa.numel(), sfb.numel(), out.stride(0), epilogue, sm_count, 0,
                 out.device.index, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("m,n,k,deal", [(8, 2048, 4096, "scratch"), (32, 4096, 8192, "scratch"),
                                        (4, 1024, 8320, "scratch"), (8, 512, 32768, "scratch as dispatched"),
                                        (8, 2048, 4096, "cluster"), (16, 7168, 2048, "whole tiles"),
                                        (20, 24576, 1536, "whole tiles")], ids=lambda v: str(v))
def test_matches_the_allocating_entry_point_twice_in_a_row(hq, monkeypatch, m, n, k, deal):
    # the cases that deal a tile to several CTAs through the scratch memory are the point of the
    # entry; the others check that it is the same kernel in every other respect
    if deal == "scratch":
        monkeypatch.setenv("HALOPS_B200_DECODE", "split,nocluster")
    tile = hq.describe_tile(m, n, k)
    if deal.startswith("scratch"):
        assert "splitk=1" in tile and "cluster=1" in tile, tile
    elif deal == "cluster":
        assert "splitk=1" in tile and "cluster=1" not in tile, tile
    else:
        assert "splitk=0" in tile, tile
    aq, bq, sfa, sfb = _operands(hq, m, n, k, seed=1000 + m)
    want = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, want, None, None, -1, "w8a8-mxfp8", False)
    assert hq.device_status() == 0
    free_before = None
    for call in range(2):
        out = torch.full([m, n], 5.0, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        if call == 1:
            free_before = torch.cuda.mem_get_info()[0]
        _noalloc(aq, bq, sfa, sfb, out)
        assert hq.device_status() == 0
        if call == 1:
            # nothing was allocated on the device by the second call (the first one may have
            # loaded the kernel's code)
            assert torch.cuda.mem_get_info()[0] == free_before
        torch.testing.assert_close(out.float(), want.float(), **TOL)
        # same kernel, same deal of the work: the very same bits
        assert torch.equal(out, want), f"call {call} differs from hq_dense_gemm"


def test_sigmoid_and_fewer_sms(hq):
    m, n, k = 8, 1024, 2048
    aq, bq, sfa, sfb = _operands(hq, m, n, k, seed=7)
    want = torch.empty([m, n], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, want, None, None, 64, "w8a8-mxfp8", False, hq.EpilogueOp.Sigmoid)
    for _ in range(2):
        out = torch.empty_like(want)
        _noalloc(aq, bq, sfa, sfb, out, epilogue=int(hq.EpilogueOp.Sigmoid), sm_count=64)
        assert hq.device_status() == 0
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=1e-2)
        assert torch.equal(out, want)


def test_sizes_beyond_the_fixed_array_are_rejected(hq):
    from halops_b200 import _native

    def call(m, n, k):
        _native.call("hq_dense_gemm_small_m_noalloc", None, None, None, None, None, m, n, k, 1 << 40, 1 << 40, n, 0,
                     -1, 0, 0, None)

    with pytest.raises(RuntimeError, match="at most 32 activation rows"):
        call(33, 1024, 1024)
    with pytest.raises(RuntimeError, match="at most 524288 weight rows"):
        call(8, 524288 + 128, 1024)
    with pytest.raises(RuntimeError, match="No dense w8a8-mxfp8 tile"):
        call(8, 1000, 1024)
    with pytest.raises(RuntimeError, match="Unsupported epilogue"):
        _native.call("hq_dense_gemm_small_m_noalloc", None, None, None, None, None, 8, 1024, 1024, 1 << 40, 1 << 40,
                     1024, 4, -1, 0, 0, None)
