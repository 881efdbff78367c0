"""Error behaviour at the boundary: misuse never aborts or faults; the first error sticks to
the context and surfaces at the next read-back, as device errors do in the reference
(crates/yaxus-model/src/lib.rs:187-197).  All failures here are made on the host."""
import numpy as np
import pytest
import torch

from oracle.check import dev, load
from yaxus_b200 import _lib
from yaxus_b200 import workloads as W
from yaxus_b200._lib import F16, F32
from yaxus_b200.backend import BackendError, CudaBackend, LayerMeta
from yaxus_b200.kvcache import PassMeta

pytestmark = pytest.mark.gpu


def test_errors_stick_until_cleared(backend):
    s = W.build("err", 1, 8, 2, F16, [40], [1])
    kv = load(backend, s)
    bad = PassMeta.from_rows([(0, 40)], [np.array([s.arena_pages + 7], np.uint32)])   # page outside the arena
    backend.begin_pass(bad)
    q = dev(backend, s.q)
    backend.attend(kv, 0, q, s.hq)        # infallible by signature
    assert backend.status() == _lib.YX_ERR_INVALID
    with pytest.raises(BackendError):
        backend.sync()                    # ... and raised at the read-back
    # later calls are refused while the error stands
    backend.begin_pass(s.meta)
    assert backend.status() == _lib.YX_ERR_INVALID
    backend.clear_error()
    backend.begin_pass(s.meta)
    backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
    backend.attend(kv, 0, q, s.hq)
    backend.sync()
    kv.close()


def test_rows_must_match_the_pass(backend):
    # cpu lib.rs:525: "attention rows differ from the pass"
    s = W.build("rows", 2, 8, 2, F32, [10], [2])
    kv = load(backend, s)
    backend.begin_pass(s.meta)
    x = torch.zeros(3, (8 + 4) * 128, device=backend.device)
    w = torch.zeros(128, device=backend.device)
    with pytest.raises(AssertionError):
        backend.attention(x, w, w, kv, 8, 1e-6, kv.layers[0])
    kv.close()


def test_bad_arguments(backend):
    with pytest.raises(BackendError):
        backend.new_kv(2, [LayerMeta()], 4, 1024, F16, head_dim=64)    # gpu lib.rs:72: head_dim must be 128
    with pytest.raises(BackendError):
        backend.new_kv(2, [LayerMeta()], 0, 1024, F16)
    s = W.build("args", 3, 8, 2, F16, [10], [1])
    kv = load(backend, s)
    fresh = CudaBackend(0)
    fresh._L.yx_attend(fresh._ctx, kv._h, 0, None, 0, 8, 0, None, 0)   # no begin_pass yet
    assert fresh.status() == _lib.YX_ERR_STATE
    fresh.clear_error()
    # a kv_slot that is not slot(pages, pos)
    m = PassMeta.from_rows([(0, 10)], s.tables)
    m.kv_slot = m.kv_slot + 1
    fresh.begin_pass(m)
    assert fresh.status() == _lib.YX_ERR_INVALID
    fresh.close()
    # hq not a multiple of hkv
    backend.begin_pass(s.meta)
    backend.attend(kv, 0, dev(backend, s.q), 7)
    assert backend.status() == _lib.YX_ERR_INVALID
    backend.clear_error()
    # position beyond max_pos (the reference asserts the RoPE table covers it, ops/attention.rs:33-36)
    kv2 = backend.new_kv(2, [LayerMeta()], 4, 100, F16)
    backend.begin_pass(PassMeta.from_rows([(0, 200)], [np.array([0, 1], np.uint32)]))
    backend.attend(kv2, 0, dev(backend, s.q), 8)
    assert backend.status() == _lib.YX_ERR_INVALID
    backend.clear_error()
    kv.close()
    kv2.close()


def test_several_passes_queue_without_a_sync(backend, oracle):
    # Pass metadata is copied at begin_pass and uploaded in stream order, so many passes can
    # be queued before any read-back (the reference's command-stream writes,
    # crates/yaxus-backend-gpu/src/dev/wgpu/mod.rs:284-294).
    from oracle.check import assert_close, oracle_step
    scen = [W.build("q", 40 + i, 8, 2, F16, [50 + 37 * i, 3 * i], [1 + i % 3, 2]) for i in range(12)]
    kvs = [load(backend, s) for s in scen]
    outs = []
    for s, kv in zip(scen, kvs):
        backend.begin_pass(s.meta)
        backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
        outs.append(backend.attend(kv, 0, dev(backend, s.q), s.hq))
    backend.sync()
    for s, o in zip(scen, outs):
        assert_close(o.cpu().numpy(), oracle_step(oracle, s), what=s.name)
    for kv in kvs:
        kv.close()


def test_a_device_wait_that_runs_out_is_an_error_not_a_hang(backend, oracle):
    # Every wait inside the kernels is bounded; when one runs out the kernel records it in the
    # context's status word and returns, and the next read-back reports YX_ERR_DEVICE.  Here a
    # one-CTA kernel waits on an mbarrier nobody arrives on, with a limit of about a millisecond
    # (no attention kernel is starved to provoke it).  The context stays usable afterwards.
    from oracle.check import assert_close, oracle_step, run_step
    rc = backend._L.yx_hook_expire_wait(backend._ctx, 2_000_000)
    assert rc == _lib.YX_OK
    with pytest.raises(BackendError) as e:
        backend.sync()
    assert e.value.code == _lib.YX_ERR_DEVICE and "code 2 at 900" in str(e.value)
    backend.clear_error()
    s = W.build("after", 5, 8, 2, F16, [300, 40], [1, 3])
    kv = load(backend, s)
    assert_close(run_step(backend, kv, s), oracle_step(oracle, s), what="after an expired wait")
    kv.close()
