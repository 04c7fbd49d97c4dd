"""CPU tests (gloo, world_size 2) of the multi-GPU host logic: request partitioning and the
column-split GEMM's all-gather + re-layout.  The GEMM itself is replaced by torch.matmul here
(a stand-in for the kernel in this test only; the GPU test exercises the real kernels)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def par():
    entry.load_package()
    import importlib
    return importlib.import_module(entry.PKG_NAME + ".parallel")


def test_partition_requests_covers_every_request_once():
    p = par()
    for world in (1, 2, 4, 8):
        seen = sorted(i for r in range(world) for i in p.partition_requests(64, world, r))
        assert seen == list(range(64))
        assert p.partition_requests(64, world, 0)[:2] == [0, world] if world < 64 else True
    assert p.partition_requests(3, 8, 5) == []
    with pytest.raises(ValueError):
        p.partition_requests(4, 2, 2)


def test_column_block():
    p = par()
    assert p.column_block(8192, 8, 3) == (3072, 1024)
    assert p.column_block(64, 1, 0) == (0, 64)
    with pytest.raises(ValueError):
        p.column_block(100, 8, 0)      # does not split evenly
    with pytest.raises(ValueError):
        p.column_block(48, 4, 0)       # blocks of 12 columns: rows not 16-byte multiples
    b = torch.arange(6 * 32).reshape(6, 32)
    assert torch.equal(p.slice_b(b, 0, 2, 1), b[:, 16:])
    assert torch.equal(p.slice_b(b.T.contiguous(), 1, 2, 1), b.T[16:, :])


def test_gather_tokens_single_process():
    p = par()
    toks = p.gather_tokens({1: np.array([5, 6]), 0: np.array([7])}, 2)
    assert [t.tolist() for t in toks] == [[7], [5, 6]]
    with pytest.raises(RuntimeError):
        p.gather_tokens({0: np.array([1])}, 2)


class _Buf:
    _next = 0x10000

    def __init__(self, shape):
        self.shape, self.ptr = shape, _Buf._next
        _Buf._next += 0x100000


class _Ctx:
    def alloc(self, shape):
        return _Buf(shape)


class _Vision:
    """Stands in for models.VisionModel: records what the request driver asks for."""
    tokens, proj_out = 729, 2048

    def __init__(self, max_crops):
        self.max_crops, self.calls = max_crops, []

    def encode(self, crops, out_ptr):
        self.calls.append(("one", crops.shape[0], out_ptr))

    def encode_images(self, images, out_ptrs):
        self.calls.append(("together", images.shape[0], list(out_ptrs)))


class _Req:
    def reset(self):
        pass


class _Text:
    """Stands in for models.TextModel: the "first token" of a request is its prompt length, the generated tokens
    count up from it unless forced."""
    dim = 2048

    def __init__(self):
        self.encoded, self.forwards, self.batches = [], [], []

    def request(self):
        return _Req()

    def text_encoder(self, ids, out_ptr):
        self.encoded.append((len(ids), out_ptr))

    def forward(self, req, base, want_hidden, want_logits, rows):
        self.forwards.append((base, rows))
        return None, None, rows

    def generate_batch(self, reqs, firsts, n_steps, forced=None):
        self.batches.append((len(reqs), list(firsts), None if forced is None else forced.copy()))
        if forced is not None:
            return forced
        return np.stack([np.arange(f + 1, f + 1 + n_steps, dtype=np.uint32) for f in firsts])


def test_serve_requests_groups_and_addresses_without_a_gpu():
    """The request driver's host logic with stand-in models: this rank's share, groups of max_streams, one embeds
    buffer per slot laid out [token 0 | 729 image rows | rest of the prompt], the images of a group encoded together
    only when each is one crop and the encoder has the capacity, forced tokens handed through per group."""
    p = par()
    rng = np.random.default_rng(0)
    lens = [3, 5, 2, 7, 4, 6, 1]
    requests = [p.Request(rng.integers(0, 256, (1, 378, 378, 3), dtype=np.uint8), np.arange(n)) for n in lens]
    requests[5] = p.Request(rng.integers(0, 256, (2, 378, 378, 3), dtype=np.uint8), np.arange(lens[5]))  # two crops
    ctx, vis, txt = _Ctx(), _Vision(max_crops=4), _Text()
    out = p.serve_requests(ctx, vis, txt, requests, world=2, rank=1, n_steps=3, max_streams=2)
    assert sorted(out) == [1, 3, 5]                       # request i -> rank i mod 2
    for i in (1, 3, 5):
        rows = lens[i] + 729
        assert out[i].tolist() == [rows, rows + 1, rows + 2, rows + 3]     # first token, then three steps
    # groups: (1, 3) together, (5) alone (a group of one, and two crops anyway)
    assert [c[0] for c in vis.calls] == ["together", "one"]
    kind, n_img, ptrs = vis.calls[0]
    assert n_img == 2 and len(ptrs) == 2
    bases = [f[0] for f in txt.forwards]
    assert ptrs == [bases[0] + 2048 * 2, bases[1] + 2048 * 2]            # image rows start after the first token's row
    # slot 0 again in the second group; its request is one row longer than the slot's buffer, which is replaced
    assert vis.calls[1][2] == bases[2] + 2048 * 2 and bases[2] != bases[0]
    assert [f[1] for f in txt.forwards] == [lens[1] + 729, lens[3] + 729, lens[5] + 729]
    # token 0 at the base, the rest of the prompt after the image rows
    assert txt.encoded[0] == (1, bases[0]) and txt.encoded[1] == (lens[1] - 1, bases[0] + 730 * 2048 * 2)
    assert [b[0] for b in txt.batches] == [2, 1]
    # a state dict carried over keeps the requests' caches and the embeds buffers (now large enough for every slot)
    state = {}
    t1, t2 = _Text(), _Text()
    p.serve_requests(ctx, _Vision(4), t1, requests, world=2, rank=1, n_steps=3, max_streams=2, state=state)
    p.serve_requests(ctx, _Vision(4), t2, requests, world=2, rank=1, n_steps=3, max_streams=2, state=state)
    assert [f[0] for f in t2.forwards] == [t1.forwards[2][0], t1.forwards[1][0], t1.forwards[2][0]]
    # capacity too small for the group: one encode per request
    vis2 = _Vision(max_crops=1)
    p.serve_requests(ctx, vis2, _Text(), requests, world=2, rank=1, n_steps=3, max_streams=2)
    assert [c[0] for c in vis2.calls] == ["one", "one", "one"]
    # forced tokens reach generate_batch per group, in slot order
    forced = {i: np.array([9, 8, 7], np.uint32) + i for i in (1, 3, 5)}
    txt3 = _Text()
    out3 = p.serve_requests(ctx, _Vision(4), txt3, requests, world=2, rank=1, n_steps=3, max_streams=2, forced=forced)
    assert txt3.batches[0][2].tolist() == [forced[1].tolist(), forced[3].tolist()]
    assert out3[3].tolist() == [lens[3] + 729] + forced[3].tolist()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = par()
    g = torch.Generator().manual_seed(5)
    M, K, N = 37, 48, 64
    a = torch.randn(M, K, generator=g)
    for layout in (0, 1):
        b = torch.randn(K, N, generator=g) if layout == 0 else torch.randn(N, K, generator=g)
        full = a @ (b if layout == 0 else b.T)
        bs = p.slice_b(b, layout, world, rank)
        block = a @ (bs if layout == 0 else bs.T)
        off, w = p.column_block(N, world, rank)
        assert torch.allclose(block, full[:, off:off + w], atol=1e-5)
        c = p.allgather_column_blocks(block)
        assert c.shape == (M, N) and torch.allclose(c, full, atol=1e-5), (rank, layout)
        # the re-layout hook sees [world, M, n]
        c2 = p.allgather_column_blocks(block, relayout=lambda gth: torch.cat(list(gth.unbind(0)), dim=1))
        assert torch.equal(c, c2)
    mine = p.partition_requests(7, world, rank)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    assert sorted(sum(gathered, [])) == list(range(7))
    # the host-side gather of the served requests' token ids: every rank ends up with all 7, in request order
    local = {i: np.arange(4, dtype=np.uint32) + 10 * i for i in mine}
    everything = p.gather_tokens(local, 7)
    assert len(everything) == 7 and all(np.array_equal(everything[i], np.arange(4) + 10 * i) for i in range(7))
    try:
        p.gather_tokens(local, 8)                       # request 7 was never served
        raise AssertionError("a missing request must be reported")
    except RuntimeError as e:
        assert "not served" in str(e)
    # the communicator id travels as a Python object from rank 0
    uid = p.share_unique_id(lambda: bytes(range(128)))
    assert uid == bytes(range(128))
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")


def test_colsplit_allgather_world2_gloo(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
