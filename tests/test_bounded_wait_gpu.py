"""The path a GEMM role takes when one of its mbarrier waits times out, exercised with
nothing in flight: a one-CTA kernel waits on a barrier that nothing arrives on, gives up
after a millisecond, records its code in the device status word and raises the abort flag
a second waiting thread leaves on.  No trap, no fault, no hang: the context stays usable
and the next GEMM is correct."""

import time

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hq():
    import halops_b200

    return halops_b200


def test_wait_gives_up_and_the_host_sees_it(hq):
    assert hq.device_status() == 0
    t0 = time.perf_counter()
    hq.selftest_bounded_wait(1000)
    with pytest.raises(RuntimeError, match=r"gave up on a bounded wait \(status 0x2:"):
        hq.device_status()
    # one millisecond of waiting, not the two seconds of the second thread's own limit
    assert time.perf_counter() - t0 < 1.0
    # read and cleared: the word is zero again
    assert hq.device_status() == 0


def test_context_stays_usable_after_a_timeout(hq):
    hq.selftest_bounded_wait(500)
    with pytest.raises(RuntimeError, match="bounded wait"):
        hq.device_status()
    g = torch.Generator().manual_seed(3)
    a = torch.randn([128, 512], generator=g).to(torch.bfloat16).cuda()
    b = torch.randn([256, 512], generator=g).to(torch.bfloat16).cuda()
    aq, sfa = hq.group_wise_quant(a)
    bq, sfb = hq.group_wise_quant(b)
    out = torch.empty([128, 256], dtype=torch.bfloat16, device="cuda")
    hq.dense_gemm(aq, bq, sfa, sfb, out)
    assert hq.device_status() == 0
    ref = oracle.dense_gemm_ref(aq, bq, sfa, sfb, "w8a8-mxfp8", out_dtype=torch.float32)
    assert (out.float().cpu() - ref).abs().max() / ref.abs().max() <= 1e-2


def test_limit_is_checked(hq):
    with pytest.raises(RuntimeError, match="limit_us must be in"):
        hq.selftest_bounded_wait(0)
    with pytest.raises(RuntimeError, match="limit_us must be in"):
        hq.selftest_bounded_wait(10_000_000)
