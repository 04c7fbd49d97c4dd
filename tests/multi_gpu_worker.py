"""Worker for the 2-GPU test of the column-split GEMM (launched with torch.distributed.run).
Checks both exchange modes against the oracle on rank 0 and against each other on every rank."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    ctx = pkg.Context(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    rng = np.random.default_rng(77)
    for (M, K, N, layout) in [(512, 1024, 2048, 1), (300, 520, 1024, 0), (1024, 2048, 4096, 1)]:
        a_h = rng.standard_normal((M, K)).astype(np.float16)
        b_h = (rng.standard_normal((K, N) if layout == 0 else (N, K)) * 0.05).astype(np.float16)
        a = torch.from_numpy(a_h).cuda()
        b = torch.from_numpy(b_h).cuda()
        bs = par.slice_b(b, layout, world, rank)
        outs = {}
        for mode in ("allgather", "fused"):
            g = par.ColSplitGemm(ctx, M, N, K, layout, mode=mode)
            for _ in range(2):                      # twice: buffers are reused
                c = g(a, bs)
            ctx.sync()
            torch.cuda.synchronize()
            outs[mode] = c.cpu().numpy().copy()
            dist.barrier()
        assert np.array_equal(outs["fused"], outs["allgather"]), f"rank {rank}: modes differ {M}x{N}x{K}"
        if rank == 0:
            from oracle import oracle
            ref = oracle.hgemm_nn(a_h, b_h) if layout == 0 else oracle.hgemm_nt(a_h, b_h)
            err = np.abs(outs["fused"].astype(np.float32) - ref.astype(np.float32)).max()
            tol = 1e-2 * np.abs(ref.astype(np.float32)).max()
            assert err <= tol, f"colsplit {M}x{N}x{K}: err {err} > {tol}"
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", flush=True)
    ctx.sync()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
