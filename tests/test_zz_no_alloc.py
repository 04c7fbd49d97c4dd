"""The allocation-free decode attention entry point, md_sdpa_single_noalloc.

Some hosts of this library cannot allocate device memory while they run (all of HBM was handed
to their own arena at start-up, or they sit in a latency-critical decode loop where the implicit
device synchronisation of cudaMalloc is not acceptable).  For them the library carries its
split-KV scratch as a built-in device array.  These tests call the entry point through the C ABI,
several times in a row on different inputs, and check every result against the oracle's
singleMaskedSDPA (attention.zig:759-811) and against the regular md_sdpa_single.
The file is collected last so that a failure here cannot hide any other test under `pytest -x`.
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


# 961 then 130: the second call leaves six of the first call's partial slots stale.  1: a single key.  128 / 129: the
# last length with one split (no merge) and the first with two.  2048: all 16 slots of the built-in array.
@pytest.mark.parametrize("lengths", [(961, 130), (2048, 1, 129, 128, 2048)])
def test_noalloc_matches_oracle_and_regular_entry_point(ctx, pkg, oracle, lengths):
    import torch
    lib = pkg.load()
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    try:
        rng = np.random.default_rng(123)
        for kv_len in lengths:             # calls in a row on one stream: the array keeps the previous contents
            qh, kh, vh = (f16_normal(rng, s) for s in ((32, 1, 64), (32, kv_len, 64), (32, kv_len, 64)))
            m = np.ones(kv_len, np.uint8)
            m[3::7] = 0
            q, k, v, mask = (torch.from_numpy(x).cuda() for x in (qh, kh, vh, m))
            ref = torch.empty((32, 1, 64), dtype=torch.float16, device="cuda")
            got = torch.zeros((32, 1, 64), dtype=torch.float16, device="cuda")
            torch.cuda.synchronize()
            ctx.sdpa_single(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), kv_len, out=ref.data_ptr())
            st, msg = _call(lib, q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), got.data_ptr(), kv_len,
                            stream.cuda_stream)
            assert st == 0, msg
            ctx.sync()
            torch.cuda.synchronize()
            assert_close_ref(got.cpu().numpy(), oracle.sdpa_single(qh, kh, vh, m), f"noalloc vs oracle kv_len={kv_len}")
            assert_close_ref(got.cpu().numpy(), ref.cpu().numpy(), f"noalloc vs md_sdpa_single kv_len={kv_len}")
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


def test_noalloc_rejects_tensors_of_another_device(ctx, pkg):
    """The kernel runs on the current device; a tensor that lives on another GPU must be refused, not dereferenced."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs a second GPU to own the foreign tensor")
    lib = pkg.load()
    here = torch.zeros(32 * 8 * 64, dtype=torch.float16, device="cuda:0")
    there = torch.zeros(32 * 8 * 64, dtype=torch.float16, device="cuda:1")
    torch.cuda.set_device(0)
    st, msg = _call(lib, here.data_ptr(), there.data_ptr(), here.data_ptr(), here.data_ptr(), here.data_ptr(), 8)
    assert st == 1 and "device 1" in msg and "device 0" in msg
