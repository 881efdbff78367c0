"""yx_attend_static: attention whose split-key scratch is built into the library's device
image, so that the call allocates nothing.  Called through the C ABI and compared with
yx_attend on the same pass, twice in a row (the scratch is reused, and nothing in it needs
clearing).  The file name sorts last so that the test also runs after every other GPU test
has used the context."""
import numpy as np
import pytest
import torch

from oracle.check import ABS_TOL, assert_close, dev, load, oracle_step
from yaxus_b200 import _lib
from yaxus_b200 import workloads as W
from yaxus_b200._lib import BF16, F16, F32
from yaxus_b200.backend import _YX_DTYPE, _ptr

pytestmark = pytest.mark.gpu


def attend_static(backend, kv, layer, q, hq, window=-1, out_dtype=torch.float32):
    out = torch.full((q.shape[0], hq * 128), float("nan"), dtype=out_dtype, device=backend.device)
    rc = backend._L.yx_attend_static(backend._ctx, kv._h, layer, _ptr(q), _YX_DTYPE[q.dtype], hq, int(window), _ptr(out),
                                     _YX_DTYPE[out.dtype])
    return rc, out


@pytest.mark.parametrize("kv_dtype,tol", [(F16, ABS_TOL), (F32, 2e-5), (BF16, ABS_TOL)])
def test_matches_attend_twice(backend, oracle, kv_dtype, tol):
    # two different passes back to back over the same scratch: a batched decode step with a
    # window, then ragged verification rows across page boundaries without one
    cases = [
        W.build("static-a", 11, 8, 2, kv_dtype, [300, 5, 127, 128, 1000, 0], [1, 1, 1, 1, 1, 1], window=200),
        W.build("static-b", 12, 8, 2, kv_dtype, [250, 126, 40], [5, 4, 3]),
    ]
    for s in cases:
        kv = load(backend, s)
        backend.begin_pass(s.meta)
        backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
        q = dev(backend, s.q)
        want = backend.to_host(backend.attend(kv, 0, q, s.hq))
        for call in range(2):
            rc, out = attend_static(backend, kv, 0, q, s.hq)
            assert rc == _lib.YX_OK, backend.last_error()
            got = backend.to_host(out)
            assert_close(got, want, abs_tol=tol, what=f"call {call} vs yx_attend")
        # The property the entry point exists for: with its output already allocated, a call takes
        # no device memory.  (The first call on a device is where the driver commits the image
        # that holds the built-in scratch, so the reading is taken after it.)
        out = torch.empty(q.shape[0], s.hq * 128, dtype=torch.float32, device=backend.device)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(backend.device)
        rc = backend._L.yx_attend_static(backend._ctx, kv._h, 0, _ptr(q), _YX_DTYPE[q.dtype], s.hq, -1, _ptr(out),
                                         _YX_DTYPE[out.dtype])
        backend.sync()
        free_after, _ = torch.cuda.mem_get_info(backend.device)
        assert rc == _lib.YX_OK and free_after == free_before, (free_before, free_after)
        assert_close(got, oracle_step(oracle, s), abs_tol=tol, what="vs oracle")
        kv.close()


def test_rejects_passes_beyond_the_scratch(backend):
    hq = 8
    rows = _lib.STATIC_MAX_ROW_HEADS // hq + 1
    s = W.build("static-big", 13, hq, 2, F16, [4], [rows])
    kv = load(backend, s)
    backend.begin_pass(s.meta)
    backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
    rc, _ = attend_static(backend, kv, 0, dev(backend, s.q), hq)
    assert rc == _lib.YX_ERR_INVALID
    assert "YX_STATIC_MAX_ROW_HEADS" in backend.last_error()
    backend.clear_error()
    # the limit itself is accepted
    s = W.build("static-max", 14, hq, 2, F16, [4], [rows - 1])
    kv2 = load(backend, s)
    backend.begin_pass(s.meta)
    backend.kv_append(kv2, 0, dev(backend, s.k_new), dev(backend, s.v_new))
    q = dev(backend, s.q)
    rc, out = attend_static(backend, kv2, 0, q, hq)
    assert rc == _lib.YX_OK, backend.last_error()
    assert_close(backend.to_host(out), backend.to_host(backend.attend(kv2, 0, q, hq)), what="at the limit")
    kv.close()
    kv2.close()
