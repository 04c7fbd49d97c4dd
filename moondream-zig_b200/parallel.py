"""Multi-GPU plumbing for the hot path: one process per GPU, torch.distributed for rendezvous only.

Two things shard (the reference has no distributed code at all, so the split is this library's):

* independent requests -> replicas.  Every GPU holds the full weights; request i runs on GPU
  i mod world (``partition_requests``).  ``serve_requests`` runs a rank's share of a list of
  requests — vision encode, 761-row prefill, greedy decode, the chain of moondream.zig:240-368 —
  with up to 8 requests decoding together as M <= 8 GEMVs; ``gather_tokens`` collects the token
  ids of all ranks on the host.  No collective on the data path.
* the column-split large GEMM -> one exchange step.  C[M,N] = A . B with N split over the ranks:
  rank r computes columns [r*N/world, (r+1)*N/world) from the full A and its slice of B, then every
  rank needs the whole C.  ``Comm`` wraps the library's communicator (md_comm_*: NCCL from a unique
  id, peer-mapped buffers, a device-side barrier); ``ColSplitGemm`` runs either form:
    - mode="allgather": tcgen05 GEMM into a contiguous [M, N/world] block, ncclAllGather, one
      re-layout kernel (md_hgemm_colsplit_allgather);
    - mode="fused": the GEMM's push warps store each finished tile into every rank's C over NVLink
      between two device-side barriers (md_hgemm_colsplit_fused); no collective, no re-layout.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

_sz = C.c_size_t
COMM_ID_BYTES = 128


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
    """All-gather the ranks' [M, N/world] blocks and lay them out as [M, N] with torch.distributed.

    The host-side statement of what md_hgemm_colsplit_allgather does after its GEMM; works on any backend (the
    CPU tests run it under gloo).  `relayout(gathered [world, M, n]) -> [M, world*n]` defaults to a permute."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n = local_block.shape
    gathered = torch.empty((world, m, n), dtype=local_block.dtype, device=local_block.device)
    dist.all_gather(list(gathered.unbind(0)), local_block.contiguous(), group=group)
    if relayout is not None:
        return relayout(gathered)
    return gathered.permute(1, 0, 2).reshape(m, world * n).contiguous()


def share_unique_id(make_id, group=None) -> bytes:
    """Rank 0 calls make_id() (128 bytes); every rank of the torch.distributed group gets them."""
    import torch.distributed as dist
    box = [make_id() if dist.get_rank(group) == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    if not isinstance(box[0], (bytes, bytearray)) or len(box[0]) != COMM_ID_BYTES:
        raise RuntimeError("the communicator id did not arrive")
    return bytes(box[0])


class Comm:
    """md_comm: the library's communicator over the ranks of a torch.distributed group (used for rendezvous only:
    rank 0's NCCL unique id is broadcast as a Python object, everything after that is the library's own)."""

    def __init__(self, ctx, group=None):
        import torch.distributed as dist
        self.ctx, self.lib = ctx, ctx.lib
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

        def make_id():
            buf = C.create_string_buffer(COMM_ID_BYTES)
            ctx._check(self.lib.md_comm_unique_id(ctx.h, buf))
            return buf.raw

        uid = share_unique_id(make_id, group) if self.world > 1 else bytes(COMM_ID_BYTES)
        h = C.c_void_p()
        ctx._check(self.lib.md_comm_init(ctx.h, C.c_char_p(uid), C.c_int(self.rank), C.c_int(self.world), C.byref(h)))
        self.h = h

    def symm_alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.ctx._check(self.lib.md_comm_symm_alloc(self.h, _sz(nbytes), C.byref(p)))
        return int(p.value)

    def symm_free(self, ptr: int):
        self.ctx._check(self.lib.md_comm_symm_free(self.h, C.c_void_p(ptr)))

    def barrier(self):
        self.ctx._check(self.lib.md_comm_barrier(self.h))

    def close(self):
        if getattr(self, "h", None):
            self.lib.md_comm_destroy(self.h)
            self.h = None


class ColSplitGemm:
    """C[M,N] = A[M,K] . B (column-split over the ranks of `comm`), result replicated on every rank."""

    def __init__(self, comm: Comm, M: int, N: int, K: int, b_layout: int, mode: str = "fused"):
        import torch
        assert mode in ("fused", "allgather")
        self.comm, self.ctx = comm, comm.ctx
        self.M, self.N, self.K, self.b_layout, self.mode = M, N, K, b_layout, mode
        self.off, self.width = column_block(N, comm.world, comm.rank)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.symm = None
        if mode == "fused":
            self.symm = comm.symm_alloc(M * N * 2)
            self.c_ptr = self.symm
        else:
            self.c = torch.empty((M, N), dtype=torch.float16, device=dev)
            self.c_ptr = self.c.data_ptr()

    def __call__(self, a, b_slice) -> int:
        """a [M,K] and this rank's slice of B (see slice_b), torch f16 CUDA tensors.  Returns the device address of
        C [M,N] (valid on the context's stream once the call returns)."""
        fn = self.ctx.lib.md_hgemm_colsplit_fused if self.mode == "fused" else self.ctx.lib.md_hgemm_colsplit_allgather
        self.ctx._check(fn(self.comm.h, C.c_void_p(a.data_ptr()), C.c_void_p(b_slice.data_ptr()), C.c_void_p(self.c_ptr),
                           _sz(self.M), _sz(self.N), _sz(self.K), C.c_int(self.b_layout)))
        return self.c_ptr

    def result(self):
        """C as a numpy array (waits for the stream)."""
        out = np.empty((self.M, self.N), np.float16)
        self.ctx._check(self.ctx.lib.md_memcpy_d2h(self.ctx.h, C.c_void_p(out.ctypes.data), C.c_void_p(self.c_ptr),
                                                   _sz(out.nbytes)))
        return out

    def close(self):
        if self.symm:
            self.comm.symm_free(self.symm)
            self.symm = None


# ----------------------------------------------------------------------------- independent requests

class Request:
    """One request of the box-scale workload: the crops of an image and the prompt's token ids."""

    def __init__(self, crops_u8: np.ndarray, prompt_ids):
        self.crops = np.ascontiguousarray(crops_u8, np.uint8)
        self.ids = np.ascontiguousarray(prompt_ids, np.uint32)
        assert self.crops.ndim == 4 and self.ids.size >= 1


def serve_requests(ctx, vision, text, requests: list, world: int, rank: int, n_steps: int, max_streams: int = 8,
                   forced: dict | None = None, state: dict | None = None) -> dict:
    """Run this rank's share of `requests` (request i -> rank i mod world) and return {index: tokens}.

    Per request, the chain of moondream.zig:240-368 with everything between the image and the token ids resident on
    the device: vision encode -> [embed(tok0), 729 image rows, embed(tok1..)] (moondream.zig:286-303) -> prefill ->
    first token -> n_steps greedy decode steps.  Up to `max_streams` (<= 8) requests decode together as M <= 8 GEMVs
    (md_text_generate_batch).  tokens = [first token, then the n_steps generated tokens].
    forced: {index: uint32 [n_steps]} feeds those tokens instead of the model's own (teacher forcing, for parity
    checks).  state: a dict reused across calls to keep the KV caches and buffers (8 x 384 MiB at full size)."""
    assert 1 <= max_streams <= 8
    mine = partition_requests(len(requests), world, rank)
    state = state if state is not None else {}
    reqs = state.setdefault("reqs", [])
    while len(reqs) < min(max_streams, len(mine)):
        reqs.append(text.request())
    dim, tokens = text.dim, vision.tokens
    assert vision.proj_out == dim
    embeds = state.setdefault("embeds", {})          # slot -> (DevBuf [rows, dim], rows)
    out: dict = {}
    for g0 in range(0, len(mine), max_streams):
        group = mine[g0:g0 + max_streams]
        bases = []
        for slot, idx in enumerate(group):
            rows = requests[idx].ids.size + tokens
            if slot not in embeds or embeds[slot][1] < rows:
                embeds[slot] = (ctx.alloc((rows, dim)), rows)
            bases.append(embeds[slot][0].ptr)
        # the images of a group go through the vision encoder together when each is one crop and the encoder has
        # the capacity (its GEMMs then see len(group) * 729 rows instead of 729); otherwise one encode per request
        together = len(group) > 1 and len(group) <= vision.max_crops and all(requests[i].crops.shape[0] == 1 for i in group)
        if together:
            vision.encode_images(np.concatenate([requests[i].crops for i in group]),
                                 out_ptrs=[b + dim * 2 for b in bases])
        firsts = []
        for slot, idx in enumerate(group):
            rq = requests[idx]
            rows = rq.ids.size + tokens
            base = bases[slot]
            text.text_encoder(rq.ids[:1], out_ptr=base)
            if not together:
                vision.encode(rq.crops, out_ptr=base + dim * 2)
            if rq.ids.size > 1:
                text.text_encoder(rq.ids[1:], out_ptr=base + (1 + tokens) * dim * 2)
            reqs[slot].reset()
            _, _, tok = text.forward(reqs[slot], base, want_hidden=False, want_logits=False, rows=rows)
            firsts.append(tok)
        f = None
        if forced is not None:
            f = np.stack([np.ascontiguousarray(forced[idx], np.uint32) for idx in group])
        toks = text.generate_batch(reqs[:len(group)], firsts, n_steps, forced=f)
        for slot, idx in enumerate(group):
            out[idx] = np.concatenate([np.array([firsts[slot]], np.uint32), toks[slot]])
    return out


def gather_tokens(local: dict, n_requests: int, group=None) -> list:
    """Every rank's {index: tokens} -> the list of all requests' tokens, on every rank (host-side gather; works on
    any torch.distributed backend, or without one when the process is alone)."""
    import torch.distributed as dist
    parts = [local]
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        parts = [None] * dist.get_world_size(group)
        dist.all_gather_object(parts, {int(k): np.asarray(v) for k, v in local.items()}, group=group)
    merged: dict = {}
    for p in parts:
        for k, v in p.items():
            if k in merged:
                raise RuntimeError(f"request {k} was served twice")
            merged[k] = v
    missing = [i for i in range(n_requests) if i not in merged]
    if missing:
        raise RuntimeError(f"requests {missing} were not served")
    return [merged[i] for i in range(n_requests)]
