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
