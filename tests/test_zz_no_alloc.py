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


@pytest.mark.parametrize("t", [A.Q4_0, A.Q8_0, A.Q4_K, A.Q5_K, A.Q6_K, A.IQ4_XS, A.IQ4_NL])
def test_the_array_filled_to_its_limits(ctx, t):
    """8 columns of 32768 values fill every part of the fixed array exactly (codes, scales, both kinds of
    block sums): a part one element short would overwrite its neighbour. Then a narrow call with other
    values on the same array."""
    k, m = 32768, 8
    rng = np.random.default_rng(900 + t)
    w = O.random_blocks(t, m, k, rng)
    for n, scale in ((8, 1.0), (1, 0.25)):
        x = (rng.normal(0, 1, size=(n, k)) * scale).astype(np.float32)
        want, got = both_ways(ctx, t, w, k, x)
        assert np.array_equal(got, want)
        assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL
    err = A.binding.C.c_int(-1)
    assert ctx.L.b200q_noalloc_device_error(0, A.binding.C.byref(err)) == A.OK and err.value == 0


def test_rows_that_are_not_16_byte_multiples(ctx):
    """Q6_K with K = 2816 (11 blocks of 210 bytes): the rows take the kernel's 2-byte loader."""
    t, k, m = A.Q6_K, 2816, 37
    rng = np.random.default_rng(12)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(5, k)).astype(np.float32)
    want, got = both_ways(ctx, t, w, k, x)
    assert np.array_equal(got, want) and rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_unevenly_spaced_dst_columns_are_refused(ctx):
    d = ctx.alloc(1 << 20)
    W = A.Tensor.weights(A.Q4_0, d, 1024, 4)
    X = A.Tensor.make(A.F32, [1024, 2, 2, 1], [4, 4096, 8192, 16384], d)
    Y = A.Tensor.make(A.F32, [4, 2, 2, 1], [4, 16, 48, 96], d)        # columns 0,1 | gap | 2,3
    assert ctx.L.b200q_mul_mat_noalloc(0, None, W, X, Y) == A.UNSUPPORTED
    assert b"evenly spaced" in ctx.L.b200q_noalloc_last_error()
    ctx.free(d)


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
