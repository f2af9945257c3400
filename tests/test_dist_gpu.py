"""Column-parallel mode on real GPUs: the test re-executes its worker under
``torch.distributed.run`` with one rank per GPU (NCCL), as the reference's own
multi-GPU tests do (tests/test_fused_all_reduce_mhc.py:181-218 there).  Each rank
computes its weight shard, the shards are all-gathered, and every rank compares
the assembled [M, N] output bit for bit with the single-GPU GEMM on the whole
weight.  Skipped with fewer than 2 GPUs."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker():
    import torch.distributed as dist

    import halops_b200 as hq
    from halops_b200.dist import ColumnParallelDenseGemm, shard_bounds, shard_quantized_weight

    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    m, n, k = 384, 1024 * world, 1024
    for mode in ("w8a8-mxfp8", "w4a4-nvfp4"):
        g = torch.Generator(device=dev).manual_seed(11)  # same seed on every rank
        x = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn([n, k], generator=g, device=dev) * 0.02).to(torch.bfloat16)
        alpha = torch.full([1], 0.5, dtype=torch.float32, device=dev) if mode == "w4a4-nvfp4" else None
        # single-GPU result on the whole weight
        xq, sfa = hq.group_wise_quant(x, mode=mode)
        wq, sfb = hq.group_wise_quant(w, mode=mode)
        want = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
        hq.dense_gemm(xq, wq, sfa, sfb, want, None, alpha, -1, mode)
        # sharded: quantise only this rank's rows ...
        start, rows = shard_bounds(n, world, rank)
        layer = ColumnParallelDenseGemm(w[start:start + rows], mode=mode)
        if alpha is not None:
            layer.set_alpha(alpha)
        got = layer(x, gather=True)
        assert torch.equal(got, want), f"rank {rank} {mode}: gathered output differs"
        # the same with the gather overlapped block by block (4 blocks of 256 rows), twice in a
        # row on the same staging buffer
        x4 = torch.randn([1024, k], generator=g, device=dev).to(torch.bfloat16)
        x4q, sfa4 = hq.group_wise_quant(x4, mode=mode)
        want4 = torch.empty([1024, n], dtype=torch.bfloat16, device=dev)
        hq.dense_gemm(x4q, wq, sfa4, sfb, want4, None, alpha, -1, mode)
        # with both transports: pushes by the copy engines into the peers' symmetric memory and NCCL
        # all-gathers per block ("auto" picks the first up to 4 ranks, the second from 8 on)
        for transport in ("copy", "nccl", "auto"):
            for i in range(2):
                staged = layer.gathered(x4q, sfa4, blocks=4, transport=transport)
                assert list(staged.shape) == [4, world, 256, rows]
                got4 = layer.gathered_as_matrix(staged)
                assert torch.equal(got4, want4), \
                    f"rank {rank} {mode} {transport}: block-wise gathered output differs (call {i})"
                # the next call may only overwrite the buffers once every rank has read them
                staged.zero_()
        # the all-gather inside the GEMM's epilogue (stores into the peers' symmetric memory),
        # twice in a row on the same outputs, with a ragged last row tile the second time round
        if mode == "w8a8-mxfp8":
            for rows_used, wanted in ((1024, want4), (1024, want4), (384, want)):
                aq, sa = (x4q, sfa4) if rows_used == 1024 else (xq, sfa)
                for i in range(2):
                    full = layer.gathered_fused(aq, sa)
                    assert torch.equal(full, wanted), \
                        f"rank {rank}: output gathered by the GEMM's own stores differs ({rows_used} rows, call {i})"
                    full.zero_()
        # ... or slice an already quantised weight (contiguous scale range)
        layer2 = ColumnParallelDenseGemm(shard_quantized_weight(wq, sfb, mode, world, rank), mode=mode)
        if alpha is not None:
            layer2.set_alpha(alpha)
        assert torch.equal(layer2.local_quantized(xq, sfa), want[:, start:start + rows])
        assert hq.device_status(dev) == 0
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("DIST_OK", world)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_column_parallel_matches_single_gpu():
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert f"DIST_OK {world}" in res.stdout


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    _worker()
