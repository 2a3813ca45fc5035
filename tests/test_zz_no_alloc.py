"""The allocation-free attention entry point (qw_attn_decode_static) against the batch path.

Some hosts of this library may not allocate device memory when they call in (their HBM is fully planned, or a stream
capture is open), so this entry point keeps the split-K partials in a static device array instead of a
caller-provided buffer.  It must give exactly the bytes the batch path gives (same kernels, same order), on two calls
in a row that reuse the shared array, and must refuse a request larger than the array.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
QH, KVH, HD = 16, 2, 256


def call_static(gpu, core, qkv, pos, sids, y, nb, layer, stride, max_pages, max_chunks):
    f = gpu.L.qw_attn_decode_static
    f.restype = C.c_int
    f.argtypes = [C.c_void_p] * 2 + [C.c_size_t] + [C.c_void_p] * 5 + [C.c_uint32] * 6 + [C.c_void_p, C.c_char_p, C.c_size_t]
    err = C.create_string_buffer(256)
    rc = f(core.q.dev_ptr, core.pool.dev_ptr, core.pool.size, core.ptab.dev_ptr, pos.dev_ptr, sids.dev_ptr, qkv.dev_ptr, y.dev_ptr,
           nb, layer, core.nlayers, stride, max_pages, max_chunks, gpu.L.qw_gpu_stream_handle(gpu.g, 0), err, 256)
    return rc, err.value.decode()


def test_static_scratch_entry_point_matches_batch_path_twice():
    from qwental_b200.gpu import Gpu
    from tests.test_gpu_attn_gdn import attn_oracle, attn_run, attn_setup
    gpu = Gpu()
    try:
        lens = [700, 5000, 31, 3000, 256, 1]
        core, d = attn_setup(gpu, lens, seed=123)
        for rows in ([0, 1, 2, 3, 4, 5], [3, 1, 5]):       # two calls in a row share the static array
            y_ref = attn_run(gpu, core, d, rows)            # batch path: qsa_prep + qsa_attn + qsa_merge; leaves q in core.q
            nb = len(rows)
            qkv, pos, sids = gpu.buf_from(d["qkv"][rows]), gpu.buf_from(d["pos"][rows]), gpu.buf_from(d["sids"][rows])
            y = gpu.buf(nb * QH * HD * 2).zero()
            mc = max((int(d["pos"][r]) + 1 + 255) // 256 for r in rows)
            rc, msg = call_static(gpu, core, qkv, pos, sids, y, nb, d["layer"], d["stride"], d["max_pages"], mc)
            assert rc == 0, msg
            got = y.download(np.float16, nb * QH * HD).reshape(nb, QH, HD)
            assert np.array_equal(got.view(np.uint16), y_ref.view(np.uint16))
            for i, r in enumerate(rows):                    # and the FP64 oracle of the same slot, at the batch path's tolerance
                ref, _ = attn_oracle(d, r)
                assert np.abs(got[i].astype(np.float64) - ref).max() < 2e-3, r
        # a request beyond the static array is refused with a clear message and launches nothing
        rc, msg = call_static(gpu, core, qkv, pos, sids, y, 64, d["layer"], d["stride"], 4096, 9)
        assert rc == -2 and "exceeds the static scratch" in msg
        # bad arguments: a layer outside the pool, more chunks than pages, no rows
        for bad in ((nb, 5, mc), (nb, d["layer"], d["max_pages"] + 1), (0, d["layer"], mc)):
            rc, msg = call_static(gpu, core, qkv, pos, sids, y, bad[0], bad[1], d["stride"], d["max_pages"], bad[2])
            assert rc == -1 and msg.startswith("qw_attn_decode_static:"), (bad, rc, msg)
    finally:
        gpu.close()


def test_static_scratch_at_its_exact_limit_and_with_a_position_beyond_the_chunks():
    """nb * max_chunks == 512 uses the whole static array: 8 slots of 64 pages.  Then the same rows with max_chunks cut to
    half of what the longest slot needs: the contract is broken by the caller, the merge must stay inside the partials
    the core wrote (the result of that slot is then the attention over its first pages; the others are unchanged)."""
    from qwental_b200.gpu import Gpu
    from tests.test_gpu_attn_gdn import attn_run, attn_setup
    gpu = Gpu()
    try:
        lens = [16383, 9000, 255, 12000, 4096, 100, 16000, 7]
        core, d = attn_setup(gpu, lens, seed=5)
        rows = list(range(8))
        y_ref = attn_run(gpu, core, d, rows)
        qkv, pos, sids = gpu.buf_from(d["qkv"]), gpu.buf_from(d["pos"]), gpu.buf_from(d["sids"])
        y = gpu.buf(8 * QH * HD * 2).zero()
        rc, msg = call_static(gpu, core, qkv, pos, sids, y, 8, d["layer"], d["stride"], d["max_pages"], 64)
        assert rc == 0, msg
        got = y.download(np.float16, 8 * QH * HD).reshape(8, QH, HD)
        assert np.array_equal(got.view(np.uint16), y_ref.view(np.uint16))
        rc, msg = call_static(gpu, core, qkv, pos, sids, y, 8, d["layer"], d["stride"], d["max_pages"], 32)
        assert rc == 0, msg
        got = y.download(np.float16, 8 * QH * HD).reshape(8, QH, HD)
        short = [r for r in rows if lens[r] + 1 <= 32 * 256]
        assert np.array_equal(got[short].view(np.uint16), y_ref[short].view(np.uint16))
        assert np.isfinite(got.astype(np.float32)).all()
    finally:
        gpu.close()
