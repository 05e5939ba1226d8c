"""GPU tests of the per-graph caches and of the failure path, through the C ABI.

The caches follow the reference's (marfrit/arcint contrib/llama.cpp/patches/
0000-01-kquant-integer-dpas.patch:670-688 activation conversion, :1264-1287 MoE route): keyed on the
tensor's identity as well as on its buffer, because a graph allocator hands one address to several
tensors in turn. The failure path is exercised in the one allowed form: a bounded wait that runs out
by design, no trap, no fault."""
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


def _x(dev, k, n, ident):
    return A.Tensor.make(A.F32, [k, n, 1, 1], [4, 4 * k], dev, ident)


@pytest.mark.parametrize("t,n", [(A.Q4_0, 1), (A.Q4_0, 5), (A.Q4_K, 3), (A.Q4_0, 40), (A.IQ4_XS, 24)])
def test_two_tensors_at_one_address_in_one_graph(ctx, t, n):
    """Layer L+1's activation lands where layer L's was (same address, shape and generation): with the
    tensors' identities in the descriptors both products must use their own contents."""
    m, k = 256, 1024
    w = make_weights(t, m, k, 300 + t)
    rng = np.random.default_rng(17 + n)
    xa = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    xb = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    dw, dx, dy = ctx.upload(w), ctx.upload(xa), ctx.alloc(n * m * 4)
    W, Y = A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dy, [m, n])
    ctx.stats_reset()
    ctx.graph_begin()
    ctx.mul_mat(W, _x(dx, k, n, 0x1000), Y)
    ga = ctx.download(dy, (n, m), np.float32)
    ctx.mul_mat(W, _x(dx, k, n, 0x1000), Y)                 # the same tensor again: cached
    # (a small per-32 product at one or two columns quantizes inside the GEMV and has no cache entry at all)
    fused = ctx.stats().get("gemv_fused_quant", 0) > 0
    assert ctx.stats().get("act_cache_hit", 0) == (0 if fused else 1)
    ctx.upload(xb, dx)                                      # another tensor of the graph at the same address
    ctx.mul_mat(W, _x(dx, k, n, 0x2000), Y)
    gb = ctx.download(dy, (n, m), np.float32)
    assert ctx.stats().get("act_cache_hit", 0) == (0 if fused else 1)
    assert rel_err(ga, O.mul_mat_f64(t, w, k, xa, True)) < TOL
    assert rel_err(gb, O.mul_mat_f64(t, w, k, xb, True)) < TOL
    for p in (dw, dx, dy):
        ctx.free(p)


def test_two_ids_tensors_at_one_address_in_one_graph(ctx):
    """The route cache: two layers' ids at one address within one generation."""
    t, n_exp, n_used, m, k, n_tok = A.Q4_K, 8, 2, 128, 512, 40
    w = np.stack([make_weights(t, m, k, 400 + e) for e in range(n_exp)])
    rb = w.shape[-1]
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, size=(n_tok, 1, k)).astype(np.float32)
    ids_a = O.route_ids(n_used, n_tok, n_exp, 11)
    ids_b = np.ascontiguousarray(ids_a[::-1])
    assert not np.array_equal(ids_a, ids_b)
    dw, dx, di, dy = ctx.upload(w), ctx.upload(x), ctx.upload(ids_a), ctx.alloc(n_tok * n_used * m * 4)
    W = A.Tensor.make(t, [k, m, n_exp, 1], [A.block_bytes(t), rb, rb * m, rb * m * n_exp], dw)
    X = A.Tensor.make(A.F32, [k, 1, n_tok, 1], [4, 4 * k, 4 * k], dx, 0x10)
    Y = A.Tensor.f32(dy, [m, n_used, n_tok])

    def ids(ident):
        return A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * n_used], di, ident)

    ctx.graph_begin()
    ctx.mul_mat_id(W, X, ids(0x20), Y)
    ga = ctx.download(dy, (n_tok, n_used, m), np.float32)
    ctx.upload(ids_b, di)
    ctx.mul_mat_id(W, X, ids(0x30), Y)
    gb = ctx.download(dy, (n_tok, n_used, m), np.float32)
    assert rel_err(ga.reshape(-1, m), O.mul_mat_id(t, w, m, k, x, ids_a, f64=True).reshape(-1, m)) < TOL
    assert rel_err(gb.reshape(-1, m), O.mul_mat_id(t, w, m, k, x, ids_b, f64=True).reshape(-1, m)) < TOL
    for p in (dw, dx, di, dy):
        ctx.free(p)


@pytest.mark.parametrize("t,n", [(A.Q4_K, 2), (A.Q8_0, 33)])
def test_capture_records_its_own_quantizer(ctx, t, n):
    """Warm up, then capture WITHOUT starting a new generation in between, then rewrite the activation:
    the replay must multiply by the new contents, i.e. the quantizer is part of the recorded graph."""
    m, k = 192, 2048
    w = make_weights(t, m, k, 500 + t)
    rng = np.random.default_rng(3)
    xa = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    xb = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    dw, dx, dy = ctx.upload(w), ctx.upload(xa), ctx.alloc(n * m * 4)
    W, X, Y = A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dx, [k, n]), A.Tensor.f32(dy, [m, n])
    ctx.graph_begin()
    ctx.mul_mat(W, X, Y)                                    # warm-up: sizes the scratch, fills the cache
    g = ctx.capture(lambda: ctx.mul_mat(W, X, Y))           # no graph_begin: the capture starts its own generation
    ctx.upload(xb, dx)
    ctx.graph_launch(g)
    got = ctx.download(dy, (n, m), np.float32)
    ctx.graph_free(g)
    assert rel_err(got, O.mul_mat_f64(t, w, k, xb, True)) < TOL
    for p in (dw, dx, dy):
        ctx.free(p)


def test_bounded_wait_runs_out_and_context_survives(ctx):
    """A device-side wait that nothing satisfies gives up after its poll limit, sets the error word and
    returns: b200q_synchronize reports B200Q_TIMEOUT once, and the next product on the same context is right."""
    ctx.sync()
    ctx.check(ctx.L.b200q_debug_wait_timeout(ctx.h, 2000))
    st = ctx.L.b200q_synchronize(ctx.h)
    assert st == A.binding.TIMEOUT
    assert b"gave up" in ctx.L.b200q_last_error(ctx.h)
    assert ctx.L.b200q_synchronize(ctx.h) == A.binding.OK          # the word was cleared
    t, m, k = A.Q4_0, 128, 1024
    w = make_weights(t, m, k, 77)
    x = np.random.default_rng(1).normal(0, 1, size=(2, k)).astype(np.float32)
    assert rel_err(ctx.run_mul_mat(t, w, k, x), O.mul_mat_f64(t, w, k, x, True)) < TOL
