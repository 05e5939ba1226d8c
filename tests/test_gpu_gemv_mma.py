"""The decode GEMV on warp-level integer MMAs (gemv_mma.cuh: Q6_K from three columns, Q4_K, Q5_K, IQ4_XS, Q4_0 and IQ4_NL
from four, Q8_0 from seven) against the oracle.

The kernel keeps the arithmetic of the reference's mv_q45_K / mv_q6_K bodies (marfrit/arcint contrib/llama.cpp/patches/
0000-01-kquant-integer-dpas.patch:3740-3874): exact integer dots per sub-block, integer sub-scales, float once per
super-block. Checked here: that the path is the one taken (counter), every column count, ragged row counts (a last
batch of fewer than eight rows), row lengths that leave the last warp's slice partly empty, the three slice widths,
rows too long for it (the dp4a kernel takes over), and that it agrees with the dp4a kernel it replaces to float rounding."""
import os

import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from gpu_util import TOL, make_weights, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = A.Context(0)
    yield c
    c.close()


def _ctx_with(**env):
    old = {k: os.environ.get(k) for k in env}
    os.environ.update({k: str(v) for k, v in env.items()})
    try:
        return A.Context(0)
    finally:
        for k, v in old.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


def _run(ctx, t, w, k, x):
    ctx.stats_reset()
    got = ctx.run_mul_mat(t, w, k, x)
    return got, ctx.stats()


# K: Q6_K rows are 16-byte multiples (the aligned path) only when K is a multiple of 2048
@pytest.mark.parametrize("t,k", [(A.Q4_K, 256), (A.Q4_K, 1280), (A.Q4_K, 4096), (A.Q4_K, 8448), (A.Q4_K, 11008), (A.Q4_K, 12288),
                                 (A.Q6_K, 2048), (A.Q6_K, 4096), (A.Q6_K, 6144), (A.Q6_K, 8192),
                                 (A.Q5_K, 256), (A.Q5_K, 4352), (A.Q5_K, 11008), (A.IQ4_XS, 512), (A.IQ4_XS, 5120), (A.IQ4_XS, 11264),
                                 (A.Q4_0, 256), (A.Q4_0, 4096), (A.Q4_0, 11008), (A.IQ4_NL, 768), (A.IQ4_NL, 4096), (A.IQ4_NL, 8448),
                                 (A.Q8_0, 256), (A.Q8_0, 3072), (A.Q8_0, 8448)])
@pytest.mark.parametrize("n", [3, 4, 5, 6, 7, 8])
def test_every_column_count_and_row_length(ctx, t, k, n):
    if n < {A.Q6_K: 3, A.Q8_0: 7}.get(t, 4):
        pytest.skip("the dp4a kernel is the faster one at this column count")
    m = 77                                                  # nine batches of eight rows and one of five
    w = make_weights(t, m, k, 60 + n)
    x = np.random.default_rng(k + n).normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = _run(ctx, t, w, k, x)
    assert st.get("gemv_mma") == 1, st
    assert np.isfinite(got).all()
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL
    assert rel_err(got, O.mul_mat(t, w, k, x)) < 1e-4      # the float form of the oracle: same integers, other summation order


@pytest.mark.parametrize("t,k", [(A.Q4_K, 4096), (A.Q6_K, 4096), (A.Q5_K, 2048), (A.IQ4_XS, 2048), (A.Q4_0, 2048), (A.IQ4_NL, 1024), (A.Q8_0, 1024)])
@pytest.mark.parametrize("m", [1, 7, 8, 9, 1000, 2371])
def test_row_counts(ctx, t, k, m):
    n = 8
    w = make_weights(t, m, k, 70 + m)
    x = np.random.default_rng(m).normal(0, 1, size=(n, k)).astype(np.float32)
    got, st = _run(ctx, t, w, k, x)
    assert st.get("gemv_mma") == 1
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


@pytest.mark.parametrize("t,k", [(A.Q4_K, 14336), (A.Q6_K, 14336), (A.Q6_K, 12288)])
def test_rows_too_long_fall_back(ctx, t, k):
    """More than twelve warps of four super-blocks (K > 12288), or a ring of eight rows beyond shared memory (Q6_K at
    K = 12288): the dp4a kernel takes the product."""
    w = make_weights(t, 40, k, 5)
    x = np.random.default_rng(1).normal(0, 1, size=(8, k)).astype(np.float32)
    got, st = _run(ctx, t, w, k, x)
    assert st.get("gemv_mma", 0) == 0 and st.get("gemv_8col") == 1
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL


@pytest.mark.parametrize("slice_", [2, 3, 4])
def test_slice_widths_and_the_dp4a_kernel_agree(ctx, slice_):
    """The slice width changes which warp holds which super-blocks, not the arithmetic: every width, and the dp4a kernel
    with the warp-MMA one switched off, must agree to float rounding on a row length that fits all of them."""
    other = _ctx_with(B200Q_GEMV_MMA_SLICE=slice_)
    plain = _ctx_with(B200Q_GEMV_MMA_MIN=99)
    try:
        for t in (A.Q4_K, A.Q6_K, A.Q5_K, A.IQ4_XS, A.Q4_0, A.IQ4_NL, A.Q8_0):
            if t == A.Q6_K and slice_ == 3:
                continue                                    # Q6_K: even widths only (a request for 3 runs 4)
            m, k, n = 203, 6144, 8
            w = make_weights(t, m, k, 9)
            x = np.random.default_rng(2).normal(0, 1, size=(n, k)).astype(np.float32)
            a, sa = _run(other, t, w, k, x)
            b, sb = _run(plain, t, w, k, x)
            assert sa.get("gemv_mma") == 1 and sb.get("gemv_mma", 0) == 0 and sb.get("gemv_stream") == 1
            assert rel_err(a, b) < 1e-4
            assert rel_err(a, O.mul_mat_f64(t, w, k, x, True)) < TOL
    finally:
        other.close()
        plain.close()


def test_inside_a_captured_graph_with_column_offsets(ctx):
    """Two products of one activation (the cache hit) captured and replayed: the kernel reads nothing it was not given."""
    t, m, k, n = A.Q4_K, 264, 4096, 6
    w = make_weights(t, m, k, 11)
    x = np.random.default_rng(3).normal(0, 1, size=(n, k)).astype(np.float32)
    dw, dx, dy1, dy2 = ctx.upload(w), ctx.upload(x), ctx.alloc(n * m * 4), ctx.alloc(n * m * 4)
    W, X = A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dx, [k, n])
    ctx.graph_begin()
    ctx.mul_mat(W, X, A.Tensor.f32(dy1, [m, n]))
    ctx.sync()

    def seq():
        ctx.mul_mat(W, X, A.Tensor.f32(dy1, [m, n]))
        ctx.mul_mat(W, X, A.Tensor.f32(dy2, [m, n]))
    g = ctx.capture(seq)
    for _ in range(3):
        ctx.graph_launch(g)
    ctx.sync()
    a, b = ctx.download(dy1, (n, m), np.float32), ctx.download(dy2, (n, m), np.float32)
    ctx.graph_free(g)
    for p in (dw, dx, dy1, dy2):
        ctx.free(p)
    assert np.array_equal(a, b)
    assert rel_err(a, O.mul_mat_f64(t, w, k, x, True)) < TOL


def test_per32_rows_that_are_not_whole_chunks_fall_back(ctx):
    """The kernel counts in chunks of 256 weights. For the 18-byte blocks a row is a 16-byte multiple exactly when it is
    whole chunks, so every aligned row qualifies and the others take the kernel for unaligned rows."""
    t, m, n = A.Q4_0, 40, 8
    for k, want in ((4352, 1), (4736, 0)):
        w = make_weights(t, m, k, 3)
        x = np.random.default_rng(4).normal(0, 1, size=(n, k)).astype(np.float32)
        got, st = _run(ctx, t, w, k, x)
        assert st.get("gemv_mma", 0) == want, (k, st)
        assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL
