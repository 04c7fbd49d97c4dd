"""Multi-GPU plumbing for the hot path: one process per GPU, torch.distributed for rendezvous.

Two things shard (the reference has no distributed code at all, so the split is this library's):

* independent requests -> replicas.  Every GPU holds the full weights; request i runs on GPU
  i mod world.  No collective on the data path (``partition_requests``).
* the column-split large GEMM -> one exchange step.  C[M,N] = A . B with N split over the ranks:
  rank r computes columns [r*N/world, (r+1)*N/world) from the full A and its slice of B, then every
  rank needs the whole C.
    - ``ColSplitGemm(mode="allgather")``: tcgen05 GEMM into a contiguous [M, N/world] block,
      NCCL all-gather of the blocks, strided re-layout into [M, N] (md_gather_colblocks).
    - ``ColSplitGemm(mode="fused")``: the GEMM epilogue stores each finished chunk into every rank's
      C through peer-mapped symmetric memory (md_hgemm_colsplit_push), then one cross-rank barrier;
      the transfer overlaps the math tile by tile and no separate collective or re-layout runs.
"""
from __future__ import annotations

import ctypes as C

_sz = C.c_size_t


def partition_requests(n_requests: int, world: int, rank: int) -> list[int]:
    """Indices of the requests rank `rank` serves: request i -> GPU i mod world."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world {world}")
    return list(range(rank, n_requests, world))


def column_block(n_cols: int, world: int, rank: int) -> tuple[int, int]:
    """(offset, width) of rank's column block; N must split into equal blocks of a multiple of 8 columns
    (16-byte rows for TMA)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world {world}")
    if n_cols % world or (n_cols // world) % 8:
        raise ValueError(f"N={n_cols} does not split into {world} blocks of a multiple of 8 columns")
    w = n_cols // world
    return rank * w, w


def slice_b(b, b_layout: int, world: int, rank: int):
    """This rank's slice of B: columns of a [K,N] matrix (b_layout 0) or rows of a [N,K] one (b_layout 1)."""
    n = b.shape[1] if b_layout == 0 else b.shape[0]
    off, w = column_block(n, world, rank)
    return (b[:, off:off + w] if b_layout == 0 else b[off:off + w, :]).contiguous()


def allgather_column_blocks(local_block, group=None, relayout=None):
    """All-gather the ranks' [M, N/world] blocks and lay them out as [M, N].

    `relayout(gathered [world, M, n]) -> [M, world*n]` defaults to a torch permute; the GPU path passes a
    function that calls md_gather_colblocks.  Works on any backend (the CPU tests run it under gloo)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n = local_block.shape
    gathered = torch.empty((world, m, n), dtype=local_block.dtype, device=local_block.device)
    dist.all_gather(list(gathered.unbind(0)), local_block.contiguous(), group=group)
    if relayout is not None:
        return relayout(gathered)
    return gathered.permute(1, 0, 2).reshape(m, world * n).contiguous()


class ColSplitGemm:
    """C[M,N] = A[M,K] . B (column-split over the ranks of `group`), result replicated on every rank."""

    def __init__(self, ctx, M: int, N: int, K: int, b_layout: int, mode: str = "fused", group=None):
        import torch
        import torch.distributed as dist
        assert mode in ("fused", "allgather")
        self.ctx, self.M, self.N, self.K, self.b_layout, self.mode, self.group = ctx, M, N, K, b_layout, mode, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.off, self.width = column_block(N, self.world, self.rank)
        dev = torch.device("cuda", torch.cuda.current_device())
        if mode == "fused":
            import torch.distributed._symmetric_memory as symm
            self.c = symm.empty((M, N), dtype=torch.float16, device=dev)
            self.hdl = symm.rendezvous(self.c, group if group is not None else dist.group.WORLD)
            peers = [int(p) for i, p in enumerate(self.hdl.buffer_ptrs) if i != self.rank]
            self.peer_arr = (C.c_void_p * max(len(peers), 1))(*peers)
            self.n_peers = len(peers)
        else:
            self.c = torch.empty((M, N), dtype=torch.float16, device=dev)
            self.block = torch.empty((M, self.width), dtype=torch.float16, device=dev)
            self.gathered = torch.empty((self.world, M, self.width), dtype=torch.float16, device=dev)

    def __call__(self, a, b_slice):
        """a [M,K] and this rank's slice of B (see slice_b), torch f16 CUDA tensors. Returns C [M,N]
        (valid on the current stream once the call returns)."""
        import torch.distributed as dist
        ctx = self.ctx
        if self.mode == "fused":
            self.hdl.barrier(channel=0)   # nobody still reads the previous C
            ctx._check(ctx.lib.md_hgemm_colsplit_push(
                ctx.h, C.c_void_p(a.data_ptr()), C.c_void_p(b_slice.data_ptr()), C.c_void_p(self.c.data_ptr()),
                _sz(self.M), _sz(self.width), _sz(self.K), C.c_int(self.b_layout), _sz(self.N), _sz(self.off),
                _sz(self.n_peers), self.peer_arr))
            self.hdl.barrier(channel=1)   # every rank's pushes have landed
            return self.c
        call = ctx.lib.md_hgemm_nn if self.b_layout == 0 else ctx.lib.md_hgemm_nt
        ctx._check(call(ctx.h, C.c_void_p(a.data_ptr()), C.c_void_p(b_slice.data_ptr()),
                        C.c_void_p(self.block.data_ptr()), _sz(self.M), _sz(self.width), _sz(self.K)))
        dist.all_gather_into_tensor(self.gathered, self.block, group=self.group)
        ctx._check(ctx.lib.md_gather_colblocks(ctx.h, C.c_void_p(self.gathered.data_ptr()),
                                               C.c_void_p(self.c.data_ptr()), _sz(self.world), _sz(self.M),
                                               _sz(self.width)))
        return self.c
