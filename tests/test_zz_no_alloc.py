"""The allocation-free decode attention entry point, md_sdpa_single_noalloc.

Some hosts of this library cannot allocate device memory while they run (all of HBM was handed
to their own arena at start-up, or they sit in a latency-critical decode loop where the implicit
device synchronisation of cudaMalloc is not acceptable).  For them the library carries its
split-KV scratch as a built-in device array.  This test calls the entry point through the C ABI
twice in a row on different inputs and checks each result against the regular md_sdpa_single.
It is collected last so that a failure here cannot hide any other test under `pytest -x`.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close_ref, f16_normal

pytestmark = pytest.mark.gpu


def _call(lib, q, k, v, mask, out, kv_len, stream=0):
    err = C.create_string_buffer(256)
    st = lib.md_sdpa_single_noalloc(C.c_void_p(q), C.c_void_p(k), C.c_void_p(v), C.c_void_p(mask), C.c_void_p(out),
                                    C.c_size_t(kv_len), C.c_void_p(stream), err, C.c_size_t(256))
    return st, err.value.decode()


def test_noalloc_matches_regular_entry_point_twice(ctx, pkg):
    import torch
    lib = pkg.load()
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    try:
        rng = np.random.default_rng(123)
        for kv_len in (961, 130):          # two calls in a row: 8 splits, then 2 (stale partials stay in the array)
            q = torch.from_numpy(f16_normal(rng, (32, 1, 64))).cuda()
            k = torch.from_numpy(f16_normal(rng, (32, kv_len, 64))).cuda()
            v = torch.from_numpy(f16_normal(rng, (32, kv_len, 64))).cuda()
            m = np.ones(kv_len, np.uint8)
            m[3::7] = 0
            mask = torch.from_numpy(m).cuda()
            ref = torch.empty((32, 1, 64), dtype=torch.float16, device="cuda")
            got = torch.zeros((32, 1, 64), dtype=torch.float16, device="cuda")
            torch.cuda.synchronize()
            ctx.sdpa_single(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), kv_len, out=ref.data_ptr())
            st, msg = _call(lib, q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), got.data_ptr(), kv_len,
                            stream.cuda_stream)
            assert st == 0, msg
            ctx.sync()
            torch.cuda.synchronize()
            assert_close_ref(got.cpu().numpy(), ref.cpu().numpy(), f"noalloc kv_len={kv_len}")
    finally:
        ctx.set_stream(None)


def test_noalloc_rejects_what_it_cannot_serve(ctx, pkg):
    import torch
    lib = pkg.load()
    d = torch.zeros(32 * 2049 * 64, dtype=torch.float16, device="cuda")
    st, msg = _call(lib, d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), 2049)
    assert st == 4 and "2048" in msg                      # MD_ERR_SEQUENCE_TOO_LONG, names the maximum
    host = np.zeros(32 * 64, np.float16)
    st, msg = _call(lib, host.ctypes.data, d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), 8)
    assert st == 1 and "device memory" in msg             # host pointers would need a staging allocation
    st, msg = _call(lib, 0, d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), 8)
    assert st == 1
