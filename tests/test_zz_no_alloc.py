"""b200q_mul_mat_noalloc, the entry point for callers that cannot allocate device memory (a host
whose own pool owns the whole GPU, a serving loop that must avoid cudaMalloc's device-wide
synchronisation): through the C ABI its output must equal b200q_mul_mat's, on two calls in a row
that share the library's fixed scratch array, and shapes beyond its stated limit must be refused.
This file sorts last on purpose, so a stop-at-first-failure run has already run everything else."""
import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from gpu_util import TOL, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = A.Context(0)
    yield c
    c.close()


def both_ways(ctx, t, w, k, x):
    """(result of b200q_mul_mat, result of b200q_mul_mat_noalloc) for the same device tensors."""
    m, n = w.shape[0], x.shape[0]
    dw, dx = ctx.upload(w), ctx.upload(x)
    dy0, dy1 = ctx.alloc(n * m * 4), ctx.alloc(n * m * 4)
    W, X = A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dx, [k, n])
    ctx.graph_begin()
    ctx.mul_mat(W, X, A.Tensor.f32(dy0, [m, n]))
    want = ctx.download(dy0, (n, m), np.float32)
    # the context is only used for memory and the reference result; the new entry point gets no
    # context, just the stream to enqueue on (the context's, so the download below is ordered after it)
    st = ctx.L.b200q_mul_mat_noalloc(0, ctx.stream(), W, X, A.Tensor.f32(dy1, [m, n]))
    assert st == A.OK, ctx.L.b200q_noalloc_last_error()
    got = ctx.download(dy1, (n, m), np.float32)
    for p in (dw, dx, dy0, dy1):
        ctx.free(p)
    return want, got


@pytest.mark.parametrize("t,k", [(A.Q4_K, 4096), (A.Q4_0, 2048), (A.Q6_K, 2048)])
def test_two_calls_in_a_row_match_mul_mat(ctx, t, k):
    rng = np.random.default_rng(k + t)
    m = 200
    w = O.random_blocks(t, m, k, rng)
    # second call: fewer columns and other values, so anything stale in the shared array would show
    for n, scale in ((8, 1.0), (3, 7.0)):
        x = (rng.normal(0, 1, size=(n, k)) * scale).astype(np.float32)
        want, got = both_ways(ctx, t, w, k, x)
        assert np.isfinite(got).all()
        assert rel_err(got, want.astype(np.float64)) < TOL
        assert np.array_equal(got, want)                     # the same two kernels: identical, in fact
        assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_limits_are_refused_with_a_message(ctx):
    d = ctx.alloc(1 << 20)
    W = A.Tensor.weights(A.Q4_0, d, 1024, 4)
    assert ctx.L.b200q_mul_mat_noalloc(0, None, W, A.Tensor.f32(d, [1024, 9]), A.Tensor.f32(d, [4, 9])) == A.UNSUPPORTED
    assert b"at most 8" in ctx.L.b200q_noalloc_last_error()
    Wk = A.Tensor.weights(A.Q4_0, d, 65536, 1)
    assert ctx.L.b200q_mul_mat_noalloc(0, None, Wk, A.Tensor.f32(d, [65536, 1]), A.Tensor.f32(d, [1, 1])) == A.UNSUPPORTED
    assert b"32768" in ctx.L.b200q_noalloc_last_error()
    assert ctx.L.b200q_mul_mat_noalloc(0, None, A.Tensor.weights(A.Q4_K, d, 300, 2), A.Tensor.f32(d, [300, 1]),
                                       A.Tensor.f32(d, [2, 1])) == A.UNSUPPORTED
    ctx.free(d)
