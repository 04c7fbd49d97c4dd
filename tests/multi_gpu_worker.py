"""Worker of the multi-GPU tests (launched with torch.distributed.run, one rank per GPU).

1. The column-split GEMM through the library's own communicator (md_comm_*): both exchange forms against each other
   bit for bit on every rank, and against the oracle on rank 0; run twice so that buffers and barriers are reused.
2. Independent requests partitioned over the ranks (serve_requests) and gathered on the host: every request's tokens
   equal the tokens a single rank produces for the same request.
"""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
from model_utils import text_weights, vision_weights  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    models = importlib.import_module(entry.PKG_NAME + ".models")
    ctx = pkg.Context(local)
    comm = par.Comm(ctx)
    rng = np.random.default_rng(77)
    for (M, K, N, layout) in [(512, 1024, 2048, 1), (300, 520, 1024, 0), (4096, 512, 4096, 1)]:
        a_h = rng.standard_normal((M, K)).astype(np.float16)
        b_h = (rng.standard_normal((K, N) if layout == 0 else (N, K)) * 0.05).astype(np.float16)
        a = torch.from_numpy(a_h).cuda()
        b = torch.from_numpy(b_h).cuda()
        bs = par.slice_b(b, layout, world, rank)
        outs = {}
        for mode in ("allgather", "fused"):
            g = par.ColSplitGemm(comm, M, N, K, layout, mode=mode)
            for _ in range(2):                      # twice: buffers and barrier epochs are reused
                g(a, bs)
            comm.barrier()
            outs[mode] = g.result()
            ctx.sync()
            dist.barrier()
            g.close()
        assert np.array_equal(outs["fused"], outs["allgather"]), f"rank {rank}: modes differ {M}x{N}x{K}"
        if rank == 0:
            from oracle import oracle
            ref = oracle.hgemm_nn(a_h, b_h) if layout == 0 else oracle.hgemm_nt(a_h, b_h)
            err = np.abs(outs["fused"].astype(np.float32) - ref.astype(np.float32)).max()
            tol = 1e-2 * np.abs(ref.astype(np.float32)).max()
            assert err <= tol, f"colsplit {M}x{N}x{K}: err {err} > {tol}"

    # independent requests: 5 requests over `world` ranks, groups of 2 streams, against one rank serving all of them
    tw = text_weights(4021, n_layers=2, hidden=1024, vocab=4096)
    vw = vision_weights(3021, n_layers=2)
    tm, vm = models.TextModel(ctx, tw), models.VisionModel(ctx, vw, max_crops=1)
    rq = np.random.default_rng(5)
    requests = [par.Request(rq.integers(0, 256, (1, 378, 378, 3), dtype=np.uint8), rq.integers(0, 4096, 32))
                for _ in range(5)]
    mine = par.serve_requests(ctx, vm, tm, requests, world, rank, n_steps=6, max_streams=2)
    assert sorted(mine) == par.partition_requests(5, world, rank)
    everything = par.gather_tokens(mine, 5)
    alone = par.serve_requests(ctx, vm, tm, requests, 1, 0, n_steps=6, max_streams=2)
    for i in range(5):
        assert np.array_equal(everything[i], alone[i]), f"rank {rank}: request {i} differs from the single-rank run"
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", flush=True)
    ctx.sync()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
