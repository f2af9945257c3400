"""Column-parallel (N-sharded) dense GEMM over the GPUs of one box.

The reference has no multi-GPU dense GEMM; this is the sharded mode of the
benchmark's largest configuration (M=16384, N=57344, K=8192 over 1/2/4/8 GPUs).
Output columns are independent, so rank r owns weight rows
``[r * N/w, (r + 1) * N/w)`` and computes ``out[:, r * N/w : (r + 1) * N/w]``
with no data-path collective.  ``N/w`` must be a multiple of 128 so that every
shard starts on an SfAtom boundary: the atoms of the swizzled scale tensor are
ordered by 128-row tile first, so a shard's scales are one contiguous byte
range of the global ``sfb`` (no re-swizzle).  An optional all-gather over NCCL
assembles the full ``[M, N]`` output on every rank; ``gathered`` overlaps it
with the GEMM by working on blocks of rows: while block ``i`` travels on a second
stream, the GEMM computes block ``i + 1``.  On GPUs with peer access the blocks
are pushed into the peers' buffers (symmetric memory) by the copy engines, which
take no SM from the GEMM; otherwise NCCL moves them and the GEMM leaves it a few
SMs.  ``gathered_fused`` does the gather inside the GEMM: the epilogue of the
2-CTA MXFP8 kernel stores every finished tile into the peers' outputs as well
as into its own, so no copy or collective follows the kernel.

One process per GPU (``torch.distributed``); the kernels run on each rank's
current stream.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from . import _native
from .gemm import dense_gemm, group_wise_quant

__all__ = ["shard_bounds", "shard_quantized_weight", "ColumnParallelDenseGemm"]


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """(first weight row, number of rows) of ``rank``'s shard."""
    if world < 1 or not 0 <= rank < world:
        raise RuntimeError(f"invalid rank {rank} for world size {world}")
    if n % world != 0 or (n // world) % 128 != 0:
        raise RuntimeError(
            f"N={n} cannot be sharded over {world} ranks: every shard must be a multiple of 128 "
            "rows so that it starts on a scale-atom boundary")
    rows = n // world
    return rank * rows, rows


def shard_quantized_weight(wq: torch.Tensor, sfb: torch.Tensor, mode: str, world: int, rank: int):
    """Views of ``rank``'s rows of a quantised weight ``[N, K or K/2]`` and of
    the matching contiguous byte range of its swizzled scales."""
    n = wq.size(0)
    start, rows = shard_bounds(n, world, rank)
    k = wq.size(1) * (1 if mode == "w8a8-mxfp8" else 2)
    kb_dim = k // _native.GROUP_SIZE[mode]
    flat = sfb.reshape(-1)
    sf = flat[start * kb_dim:(start + rows) * kb_dim].view(rows, kb_dim)
    return wq[start:start + rows], sf


class SymmetricMemoryUnavailable(RuntimeError):
    """The peers' buffers cannot be mapped (no peer access, or no symmetric memory in this torch)."""


class ColumnParallelDenseGemm:
    """``y = x @ W^T`` with ``W`` sharded by rows (output columns) over a process group.

    Args:
        weight: this rank's ``[N/w, K]`` bf16/fp16 weight shard (quantised here once),
            or a tuple ``(wq, sfb)`` of an already quantised shard.
        mode: quantisation recipe of both operands.
        group: process group (default: the world group); ``None`` world of 1 needs no
            initialised process group.
        gemm_fn / quant_fn: the kernels to call (defaults: this package's); tests of the
            host-side logic on CPU ranks inject stand-ins.
    """

    def __init__(self, weight, mode: str = "w8a8-mxfp8", group=None,
                 gemm_fn: Optional[Callable] = None, quant_fn: Optional[Callable] = None):
        import torch.distributed as dist

        self.mode = mode
        self._dist = dist if dist.is_available() and dist.is_initialized() else None
        self.group = group
        self.world = self._dist.get_world_size(group) if self._dist else 1
        self.rank = self._dist.get_rank(group) if self._dist else 0
        self._gemm = gemm_fn or dense_gemm
        self._quant = quant_fn or group_wise_quant
        if isinstance(weight, tuple):
            self.wq, self.sfb = weight
        else:
            self.wq, self.sfb = self._quant(weight, mode=mode)
        self.n_local = self.wq.size(0)
        if self.n_local % 128 != 0:
            raise RuntimeError("a weight shard must have a multiple of 128 rows")
        self.alpha = None
        self._staging = None
        self._blocks = None
        self._comm_stream = None
        self._symm = None   # ((shape, device), local staging, [views of every rank's staging])
        self._flag = None
        self._symm_matrix = None   # ((M, device), local [M, N], every rank's view, their addresses)

    def set_alpha(self, alpha: torch.Tensor) -> None:
        """Per-tensor float32 ``[1]`` factor of the NVFP4 recipe."""
        self.alpha = alpha

    def local(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """This rank's ``[M, N/w]`` column block from bf16/fp16 activations."""
        xq, sfa = self._quant(x, mode=self.mode)
        return self.local_quantized(xq, sfa, out)

    def local_quantized(self, xq, sfa, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = xq.size(0)
        if out is None:
            out = torch.empty([m, self.n_local], dtype=torch.bfloat16, device=xq.device)
        self._gemm(xq, self.wq, sfa, self.sfb, out, None, self.alpha, -1, self.mode)
        return out

    def gather(self, out_local: torch.Tensor) -> torch.Tensor:
        """All-gather of the column blocks: returns ``[world, M, N/w]`` (block r is
        rank r's columns) without a re-tiling pass; ``as_matrix`` gives ``[M, N]``."""
        if self.world == 1:
            return out_local.unsqueeze(0)
        m = out_local.size(0)
        shape = [self.world, m, self.n_local]
        if self._staging is None or list(self._staging.shape) != shape or self._staging.device != out_local.device:
            self._staging = torch.empty(shape, dtype=out_local.dtype, device=out_local.device)
        self._dist.all_gather_into_tensor(self._staging.view(self.world * m, self.n_local),
                                          out_local.contiguous(), group=self.group)
        return self._staging

    # ------------------------------------------------------------------ overlapped all-gather

    @staticmethod
    def default_comm_sms(world: int) -> int:
        """SMs the GEMM leaves free while an all-gather runs beside it.  NCCL's kernels need
        SMs of their own: the GEMM is persistent with one CTA per SM that takes all of the
        SM's shared memory, so nothing else becomes resident next to it."""
        return 0 if world <= 1 else (8 if world == 2 else 16)

    def _symmetric_staging(self, shape, device):
        """Staging buffer of ``gathered`` in symmetric memory: the same allocation on every
        rank, each mapped into every other rank's address space, so a rank can push its
        blocks into its peers' buffers with plain device-to-device copies (copy engines over
        NVLink, no SM).  Collective: every rank calls it with the same shape.  Returns None
        where symmetric memory cannot be had; the caller then gathers with NCCL."""
        if self._symm is not None and self._symm[0] == (tuple(shape), device):
            return self._symm[1], self._symm[2]
        try:
            import torch.distributed._symmetric_memory as symm

            group = self.group if self.group is not None else self._dist.group.WORLD
            local = symm.empty(shape, dtype=torch.bfloat16, device=device)
            handle = symm.rendezvous(local, group)
            peers = [handle.get_buffer(r, shape, torch.bfloat16) for r in range(self.world)]
        except Exception:  # no peer access / no symmetric memory in this build: NCCL it is
            self._symm = ((tuple(shape), device), None, None)
            return None, None
        self._symm = ((tuple(shape), device), local, peers)
        self._flag = torch.zeros([1], dtype=torch.int32, device=device)
        return local, peers

    def _rendezvous_on(self, stream) -> None:
        """All ranks meet, in the order of ``stream``: a one-element NCCL all-reduce."""
        with torch.cuda.stream(stream):
            self._dist.all_reduce(self._flag, group=self.group)

    def gathered(self, xq: torch.Tensor, sfa: torch.Tensor, blocks: int = 8,
                 comm_sms: Optional[int] = None, transport: str = "auto", compute: bool = True) -> torch.Tensor:
        """GEMM and all-gather overlapped.  The rows of the activation are cut into
        ``blocks`` blocks (each a multiple of 128 rows, so a block's scales are a contiguous
        byte range of ``sfa``, and at least 256 rows, so a block runs on the same multi-row-tile
        kernels as the whole activation would and the result keeps its bits: the small-M and
        split-K kernels add partial sums in another order).  While the GEMM computes block
        ``i + 1`` on the current stream, block ``i`` travels on a second stream:

        * ``transport="copy"`` (what ``"auto"`` picks for up to 4 ranks with peer access): the staging
          buffer lives in symmetric memory and every rank pushes its block into its peers'
          buffers with device-to-device copies, which the copy engines carry over NVLink
          without taking an SM from the GEMM.  Two small NCCL all-reduces fence the pushes: one
          before the first push (every rank is done reading the previous call's result) and one
          after the last (everybody's pushes have landed).
        * ``transport="nccl"`` (``"auto"`` from 8 ranks on): ``all_gather_into_tensor`` per block; its
          kernels need SMs, so the GEMM runs on a grid that leaves ``comm_sms`` SMs free.

        Returns ``[blocks, world, M / blocks, N/w]``: entry ``[b, r]`` holds rows
        ``[b M / blocks, (b + 1) M / blocks)`` of rank ``r``'s columns; ``gathered_as_matrix``
        turns it into ``[M, N]`` with one copy.  The current stream waits for the transfers
        before it runs anything queued after this call.  Collective: every rank calls it.
        ``compute=False`` skips the GEMMs and moves what the staging buffer holds (to time the
        transfers alone)."""
        m = xq.size(0)
        while blocks > 1 and (m % blocks != 0 or (m // blocks) % 128 != 0 or m // blocks < 256):
            blocks -= 1
        rows = m // blocks
        shape = [blocks, self.world, rows, self.n_local]
        on_gpu = xq.is_cuda
        peers = None
        # "auto": the copy engines up to 4 ranks; from 8 ranks on NCCL's all-gathers move more bytes
        # per second than pushes of a block to seven peers in turn (581 against 465 GB/s into a
        # rank on 8 B200; pushes on several streams at once were slower still)
        if transport == "auto":
            transport = "copy" if self.world <= 4 else "nccl"
        if on_gpu and self.world > 1 and transport == "copy":
            staging, peers = self._symmetric_staging(shape, xq.device)
            # (without peer access or symmetric memory in this build: NCCL it is)
        if peers is None:
            if self._blocks is None or list(self._blocks.shape) != shape or self._blocks.device != xq.device:
                self._blocks = torch.empty(shape, dtype=torch.bfloat16, device=xq.device)
            staging = self._blocks
        kb_dim = sfa.numel() // ((m + 127) // 128 * 128)
        sfa_flat = sfa.reshape(-1)
        sms = -1
        comm = cur = None
        if on_gpu and self.world > 1:
            if peers is None:
                comm_sms = self.default_comm_sms(self.world) if comm_sms is None else comm_sms
                total = torch.cuda.get_device_properties(xq.device).multi_processor_count
                sms = max(2, total - comm_sms)
            if self._comm_stream is None or self._comm_stream.device != xq.device:
                self._comm_stream = torch.cuda.Stream(xq.device, priority=-1)
            comm = self._comm_stream
            cur = torch.cuda.current_stream(xq.device)
            # the transfers come after everything queued on the current stream so far, the
            # readers of the previous call's result among it
            comm.wait_stream(cur)
            if peers is not None:
                # ... on every rank: nobody pushes into a buffer that is still being read
                self._rendezvous_on(comm)
        for b in range(blocks):
            mine = staging[b, self.rank]
            # (a single block may have any number of rows: it takes the whole, padded scale tensor)
            block_sfa = sfa if blocks == 1 else sfa_flat[b * rows * kb_dim:(b + 1) * rows * kb_dim].view(rows, kb_dim)
            if compute:
                self._gemm(xq[b * rows:(b + 1) * rows], self.wq, block_sfa, self.sfb, mine, None, self.alpha, sms,
                           self.mode)
            if self.world == 1:
                continue
            flat = staging[b].view(self.world * rows, self.n_local)
            if comm is None:
                self._dist.all_gather_into_tensor(flat, mine, group=self.group)
                continue
            done = torch.cuda.Event()
            done.record(cur)
            comm.wait_event(done)
            with torch.cuda.stream(comm):
                if peers is None:
                    # in place: rank r's input is block r of the output
                    self._dist.all_gather_into_tensor(flat, mine, group=self.group)
                else:
                    # at any moment every rank pushes to a different peer
                    for i in range(1, self.world):
                        peers[(self.rank + i) % self.world][b, self.rank].copy_(mine, non_blocking=True)
        if comm is not None:
            if peers is not None:
                # once every rank is past this point, every push has landed
                self._rendezvous_on(comm)
            cur.wait_stream(comm)
        return staging

    # ------------------------------------------------------------------ all-gather inside the GEMM

    def fused_supported(self, m: int) -> bool:
        """Whether ``gathered_fused`` can run: MXFP8 on the 2-CTA 256 x 256 tile, at most 8 ranks."""
        return (self.mode == "w8a8-mxfp8" and self.alpha is None and self.n_local % 256 == 0 and m > 128
                and 1 <= self.world <= 8)

    def _symmetric_matrix(self, m: int, device):
        """The ``[M, N]`` output of ``gathered_fused`` in symmetric memory, with the device
        addresses of every rank's copy as this process sees them.  Collective."""
        key = (m, device)
        if self._symm_matrix is not None and self._symm_matrix[0] == key:
            return self._symm_matrix[1:]
        import ctypes

        shape = [m, self.world * self.n_local]
        if self.world == 1:
            local = torch.empty(shape, dtype=torch.bfloat16, device=device)
            views = [local]
        else:
            try:
                import torch.distributed._symmetric_memory as symm

                group = self.group if self.group is not None else self._dist.group.WORLD
                local = symm.empty(shape, dtype=torch.bfloat16, device=device)
                handle = symm.rendezvous(local, group)
                views = [handle.get_buffer(r, shape, torch.bfloat16) for r in range(self.world)]
            except Exception as ex:  # no peer access / no symmetric memory in this build
                raise SymmetricMemoryUnavailable(str(ex)) from ex
            if self._flag is None:
                self._flag = torch.zeros([1], dtype=torch.int32, device=device)
        addresses = (ctypes.c_void_p * self.world)(*[v.data_ptr() for v in views])
        self._symm_matrix = (key, local, views, addresses)
        return local, views, addresses

    def gathered_fused(self, xq: torch.Tensor, sfa: torch.Tensor, sm_count: int = -1) -> torch.Tensor:
        """GEMM and all-gather in ONE kernel.  Every rank holds an ``[M, N]`` output in symmetric
        memory; the GEMM's epilogue stages each finished piece of a tile in shared memory once and
        stores it, with one TMA store per matrix, into this rank's columns of its own output and
        of every peer's output (over NVLink), so the transfer of a tile runs while the tensor
        cores work on the next one and no copy or collective kernel follows.  All loads
        (operands, scales) are from this GPU's memory.  Two one-element NCCL all-reduces fence
        the call on the current stream: before the kernel (no rank still reads the previous
        result) and after it (every rank's stores are complete).  Returns this rank's ``[M, N]``
        matrix, valid on the current stream; the next call overwrites it.  Collective."""
        m, k = xq.shape
        if not self.fused_supported(m):
            raise RuntimeError("gathered_fused needs the MXFP8 recipe, a shard with a multiple of 256 rows, more "
                               "than 128 activation rows and at most 8 ranks")
        local, _views, addresses = self._symmetric_matrix(m, xq.device)
        stream = torch.cuda.current_stream(xq.device)
        if self.world > 1:
            self._dist.all_reduce(self._flag, group=self.group)
        _native.call("hq_dense_gemm_allgather", xq.data_ptr(), self.wq.data_ptr(), sfa.data_ptr(), self.sfb.data_ptr(),
                     addresses, self.world, self.rank, m, self.n_local, k, sfa.numel(), self.sfb.numel(),
                     local.stride(0), sm_count, 0, xq.device.index, stream.cuda_stream)
        if self.world > 1:
            self._dist.all_reduce(self._flag, group=self.group)
        return local

    @staticmethod
    def gathered_as_matrix(staging: torch.Tensor) -> torch.Tensor:
        """``[blocks, world, rows, N/w]`` -> ``[M, N]`` (one copy)."""
        b, w, rows, nl = staging.shape
        return staging.permute(0, 2, 1, 3).reshape(b * rows, w * nl)

    @staticmethod
    def as_matrix(gathered: torch.Tensor) -> torch.Tensor:
        """``[world, M, N/w]`` -> ``[M, N]`` (one copy)."""
        w, m, nl = gathered.shape
        return gathered.permute(1, 0, 2).reshape(m, w * nl)

    def __call__(self, x: torch.Tensor, gather: bool = False, overlap: bool = False) -> torch.Tensor:
        if gather and overlap:
            xq, sfa = self._quant(x, mode=self.mode)
            if xq.is_cuda and self.world > 1 and self.fused_supported(xq.size(0)):
                # (on 2, 4 and 8 B200 the GEMM that gathers in its epilogue gave the shortest step)
                try:
                    return self.gathered_fused(xq, sfa)
                except SymmetricMemoryUnavailable:  # on every rank alike: the block-wise overlap it is
                    pass
            return self.gathered_as_matrix(self.gathered(xq, sfa))
        out = self.local(x)
        return self.as_matrix(self.gather(out)) if gather else out
