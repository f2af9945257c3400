"""Host-side logic of the column-parallel mode on CPU ranks (gloo, world size 2):
shard bounds, the contiguous scale range of a shard, gather layout.  The GPU
kernels are replaced by injected stand-ins (the library itself has no CPU path)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def test_shard_bounds():
    from halops_b200.dist import shard_bounds

    assert shard_bounds(57344, 8, 3) == (3 * 7168, 7168)
    assert shard_bounds(57344, 1, 0) == (0, 57344)
    with pytest.raises(RuntimeError, match="multiple of 128"):
        shard_bounds(1000, 2, 0)
    with pytest.raises(RuntimeError, match="multiple of 128"):
        shard_bounds(384, 2, 0)  # 192-row shards would start inside a scale atom
    with pytest.raises(RuntimeError, match="invalid rank"):
        shard_bounds(1024, 2, 2)


@pytest.mark.parametrize("mode", ["w8a8-mxfp8", "w4a4-nvfp4"])
def test_shard_scales_are_a_contiguous_range(mode):
    """Swizzled scales of a 128-row-aligned shard == swizzle of the shard alone."""
    from halops_b200.dist import shard_quantized_weight

    g = torch.Generator().manual_seed(1)
    w = torch.randn([512, 256], generator=g).to(torch.bfloat16)
    q, sf = oracle.quant_group_wise(w, mode)
    for rank in range(2):
        qs, sfs = shard_quantized_weight(torch.from_numpy(q), torch.from_numpy(sf), mode, 2, rank)
        q_alone, sf_alone = oracle.quant_group_wise(w[rank * 256:(rank + 1) * 256], mode)
        assert np.array_equal(qs.numpy(), q_alone)
        assert np.array_equal(sfs.numpy(), sf_alone)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from halops_b200.dist import ColumnParallelDenseGemm, shard_bounds

        m, n, k = 64, 512, 256
        g = torch.Generator().manual_seed(7)
        x = torch.randn([m, k], generator=g).to(torch.bfloat16)
        w = torch.randn([n, k], generator=g).to(torch.bfloat16)
        start, rows = shard_bounds(n, world, rank)

        def quant(t, mode="w8a8-mxfp8", **_):
            q, sf = oracle.quant_group_wise(t, mode)
            return torch.from_numpy(q), torch.from_numpy(sf)

        def gemm(xq, wq, sfa, sfb, out, bias, alpha, sm, mode, *_):
            out.copy_(oracle.dense_gemm_ref(xq, wq, sfa, sfb, mode))

        layer = ColumnParallelDenseGemm(w[start:start + rows], gemm_fn=gemm, quant_fn=quant)
        assert (layer.world, layer.rank, layer.n_local) == (world, rank, rows)
        full = layer(x, gather=True)
        xq, sfa = quant(x)
        wq, sfb = quant(w)
        want = oracle.dense_gemm_ref(xq, wq, sfa, sfb, "w8a8-mxfp8")
        ok = bool(torch.equal(full, want)) and list(layer.gather(layer.local(x)).shape) == [world, m, rows]
        # the block-wise (overlapped on a GPU) gather: one block here, since 64 rows cannot be cut
        ok = ok and bool(torch.equal(layer(x, gather=True, overlap=True), want))
        # ... and two blocks of 256 rows (the smallest allowed), each with its own contiguous
        # range of scale bytes
        x2 = torch.randn([512, k], generator=g).to(torch.bfloat16)
        x2q, sfa2 = quant(x2)
        staged = layer.gathered(x2q, sfa2, blocks=8)
        ok = ok and list(staged.shape) == [2, world, 256, rows]
        ok = ok and bool(torch.equal(layer.gathered_as_matrix(staged), oracle.dense_gemm_ref(x2q, wq, sfa2, sfb, "w8a8-mxfp8")))
        # the GEMM that gathers in its epilogue applies to this shard from 129 rows on, but only on a
        # GPU: here the overlapped call takes the block-wise path and gives the same matrix
        ok = ok and layer.fused_supported(512) and not layer.fused_supported(64)
        ok = ok and bool(torch.equal(layer(x2, gather=True, overlap=True),
                                     oracle.dense_gemm_ref(x2q, wq, sfa2, sfb, "w8a8-mxfp8")))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_column_parallel_gather_world2():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(ret) == {0: True, 1: True}
