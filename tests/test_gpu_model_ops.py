"""The operators of the Backend trait either side of attention (crates/yaxus-model/src/lib.rs:124-171)
against the CPU oracle's restatement of the CPU backend (crates/yaxus-backend-cpu/src/lib.rs:485-562)."""
import numpy as np
import pytest
import torch

from yaxus_b200.kvcache import PassMeta

pytestmark = pytest.mark.gpu


def dev(backend, x):
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(backend.device)


def bf16_to_f32(bits):
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def assert_matmul_close(got, x, w_bits, ref, tol=1e-4):
    # The reference's own bound (cpu lib.rs:736-740): tol x the sum of the terms' magnitudes.
    scale = np.abs(x.astype(np.float64)) @ np.abs(bf16_to_f32(w_bits).astype(np.float64)).T
    err = np.abs(got.astype(np.float64) - ref)
    assert (err <= tol * np.maximum(scale, 1.0)).all(), float((err / np.maximum(scale, 1.0)).max())


def test_reference_matmul_test(backend, oracle):
    # matmul_matches_a_plain_loop (cpu lib.rs:716-744), bf16 arm, same generator and seeds.
    n, k = 40, 64
    w_bits = oracle.to_bf16(oracle.values(n * k, 7)).reshape(n, k)
    w = backend.load_weight(w_bits)
    for t in (1, 3, 9):
        x = oracle.values(t * k, t).reshape(t, k)
        got = backend.to_host(backend.matmul(dev(backend, x), w))
        assert got.shape == (t, n)
        assert_matmul_close(got, x, w_bits, oracle.matmul(x, w_bits))


@pytest.mark.parametrize("t,n,k", [(1, 256, 1024), (16, 1000, 2048), (5, 129, 96), (16, 4096, 4096), (33, 512, 3072),
                                   (80, 384, 1024), (7, 64, 40), (512, 1536, 2048), (3, 40, 128)])
def test_matmul_shapes(backend, oracle, t, n, k):
    # decode-sized passes over model-sized weights, passes of more than 32 rows (cuBLASLt; and the
    # row kernel taking them 32 at a time, which is what runs where that library is missing),
    # ragged N, K off the tensor-core kernel's 128 (the warp-per-output kernel)
    rng = np.random.default_rng(t * 1000 + n)
    x = rng.standard_normal((t, k)).astype(np.float32)
    w_bits = oracle.to_bf16((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
    w = backend.load_weight(w_bits)
    ref = oracle.matmul(x, w_bits)
    got = backend.to_host(backend.matmul(dev(backend, x), w))
    assert_matmul_close(got, x, w_bits, ref, tol=2e-5)
    if t > 32:
        backend.set_tuning(force_path=2)
        got = backend.to_host(backend.matmul(dev(backend, x), w))
        backend.set_tuning()
        assert_matmul_close(got, x, w_bits, ref, tol=2e-5)


@pytest.mark.parametrize("t,inner,k", [(16, 1024, 2048), (3, 100, 64), (40, 256, 512)])
def test_matmul_glu_is_matmul_then_swiglu(backend, oracle, t, inner, k):
    rng = np.random.default_rng(inner)
    x = rng.standard_normal((t, k)).astype(np.float32)
    w_bits = oracle.to_bf16((rng.standard_normal((2 * inner, k)) / np.sqrt(k)).astype(np.float32))
    w = backend.load_weight(w_bits)
    got = backend.to_host(backend.matmul_glu(dev(backend, x), w))
    ref = oracle.swiglu(oracle.matmul(x, w_bits))
    assert got.shape == (t, inner)
    assert np.abs(got - ref).max() <= 2e-5 * max(1.0, float(np.abs(ref).max()))
    two = backend.to_host(backend.swiglu(backend.matmul(dev(backend, x), w)))
    assert np.abs(two - ref).max() <= 2e-5 * max(1.0, float(np.abs(ref).max()))


@pytest.mark.parametrize("rows,cols", [(1, 128), (16, 4096), (5, 1000), (80, 2048)])
def test_rmsnorm_and_add_norm(backend, oracle, rows, cols):
    rng = np.random.default_rng(cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 3
    d = rng.standard_normal((rows, cols)).astype(np.float32)
    w1 = oracle.to_bf16(rng.standard_normal(cols).astype(np.float32) * 0.1)
    w2 = oracle.to_bf16(rng.standard_normal(cols).astype(np.float32) * 0.1)
    pw, qw = backend.load_weight(w1), backend.load_weight(w2)     # vectors: widened to f32 at load
    assert pw.dtype == torch.float32
    ref = oracle.rmsnorm(x, bf16_to_f32(w1), 1.0, 1e-6)
    got = backend.to_host(backend.rmsnorm(dev(backend, x), pw, 1.0, 1e-6))
    assert np.abs(got - ref).max() <= 1e-5 * max(1.0, float(np.abs(ref).max()))
    # add_norm: x is updated in place, the return is the pre-norm of the next block
    xd = dev(backend, x)
    out = backend.add_norm(xd, dev(backend, d), pw, 0.0, qw, 1.0, 1e-6)
    x_ref, out_ref = oracle.add_norm(x, d, bf16_to_f32(w1), 0.0, bf16_to_f32(w2), 1.0, 1e-6)
    assert np.abs(backend.to_host(xd) - x_ref).max() <= 1e-5 * max(1.0, float(np.abs(x_ref).max()))
    assert np.abs(backend.to_host(out) - out_ref).max() <= 2e-5 * max(1.0, float(np.abs(out_ref).max()))


def test_embed_select_add(backend, oracle):
    rng = np.random.default_rng(2)
    table_bits = oracle.to_bf16(rng.standard_normal((300, 256)).astype(np.float32))
    table = backend.load_weight(table_bits)
    ids = np.array([7, 299, 0, 7, 123], np.uint32)
    meta = PassMeta.from_rows([(0, p) for p in range(5)], [np.array([2])])
    meta.ids = ids
    backend.begin_pass(meta)
    e = backend.embed(table)
    assert np.array_equal(backend.to_host(e), oracle.embed(table_bits, ids))        # bit-exact: a gather
    sel = backend.select_rows(e, [4, 0, 0])
    assert np.array_equal(backend.to_host(sel), oracle.embed(table_bits, ids)[[4, 0, 0]])
    a, b = rng.standard_normal((5, 256)).astype(np.float32), rng.standard_normal((5, 256)).astype(np.float32)
    ad = dev(backend, a)
    backend.add_assign(ad, dev(backend, b))
    assert np.array_equal(backend.to_host(ad), a + b)                                 # one rounding each
    assert backend.weight_bytes() >= table_bits.size * 2


def test_argmax_rows(backend, oracle):
    # argmax_takes_the_first_maximum_and_skips_nans (cpu lib.rs:746-752), then vocabulary-sized rows
    nan = np.nan
    for row, want in [([1.0, 3.0, 3.0, 2.0], 1), ([nan, 1.0, 2.0], 2), ([0.5, nan, 0.2], 0), ([nan, nan], 0)]:
        assert int(backend.argmax_rows(dev(backend, np.array([row], np.float32)))[0]) == want
    rng = np.random.default_rng(4)
    x = rng.standard_normal((16, 100003)).astype(np.float32)
    x[3, 500] = x[3, 90000] = 50.0           # a tie: the first one
    x[5, :] = np.nan
    x[6, 17] = np.inf
    x[7, :] = -np.inf                        # nothing is larger than -inf: 0
    got = backend.argmax_rows(dev(backend, x))
    assert np.array_equal(got, oracle.argmax_rows(x))
    assert got[3] == 500 and got[5] == 0 and got[6] == 17 and got[7] == 0


def test_bad_indices_are_refused_on_the_host(backend, oracle):
    table = backend.load_weight(oracle.to_bf16(np.ones((4, 32), np.float32)))
    meta = PassMeta.from_rows([(0, 0)], [np.array([0])])
    meta.ids = np.array([4], np.uint32)      # one past the table
    backend.begin_pass(meta)
    backend.embed(table)
    assert backend.status() != 0 and "token id" in backend.last_error()
    backend.clear_error()
    backend.select_rows(torch.zeros(2, 8, device=backend.device), [2])
    assert backend.status() != 0 and "row index" in backend.last_error()
    backend.clear_error()
