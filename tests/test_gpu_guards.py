"""Guard words around the library's scratch and around the caller's output, checked on the host.

The pool this runs on offers no device-side memory checker, so out-of-bounds writes are looked for the plain way:
a context created with B200Q_CANARY=1 allocates every scratch block (quantized activations, route tables, split-K and
MoE scratch) at exactly the size asked for with 256 guard bytes either side, and the outputs here carry a guard row of
their own. Ragged row counts and every column-count branch (decode GEMV 1..8, the small-batch kernel, the tensor-core
tiles, the routed forms) run, then the guards must be untouched and the results equal to a plain context's."""
import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from gpu_util import make_weights

pytestmark = pytest.mark.gpu

GUARD = 0x7FC5C5C5          # a NaN pattern no product writes


@pytest.fixture(scope="module")
def ctxs():
    import os
    old = os.environ.get("B200Q_CANARY")
    os.environ["B200Q_CANARY"] = "1"
    try:
        guarded = A.Context(0)
    finally:
        if old is None:
            del os.environ["B200Q_CANARY"]
        else:
            os.environ["B200Q_CANARY"] = old
    plain = A.Context(0)
    yield guarded, plain
    guarded.close()
    plain.close()


def _guarded_out(ctx, n_words):
    host = np.full(n_words + 64, GUARD, np.uint32)
    return ctx.upload(host), host


def _product(ctx, t, w, m, k, x):
    n = x.shape[0]
    dw, dx = ctx.upload(w), ctx.upload(x)
    dy, _ = _guarded_out(ctx, n * m)
    ctx.graph_begin()
    ctx.mul_mat(A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dx, [k, n]), A.Tensor.f32(dy, [m, n]))
    raw = ctx.download(dy, (n * m + 64,), np.uint32)
    for p in (dw, dx, dy):
        ctx.free(p)
    return raw[:n * m].view(np.float32).reshape(n, m), raw[n * m:]


@pytest.mark.parametrize("t", [A.Q4_0, A.Q8_0, A.Q4_K, A.Q5_K, A.Q6_K, A.IQ4_NL, A.IQ4_XS])
def test_products_leave_every_guard_untouched(ctxs, t):
    guarded, plain = ctxs
    k = 1280                                        # Q6_K / IQ4_XS rows that are not 16-byte multiples
    for m, n in ((200, 1), (331, 3), (200, 8), (77, 9), (200, 40), (331, 130), (1000, 520)):
        w = make_weights(t, m, k, 40 + m + n)
        x = np.random.default_rng(m * n).normal(0, 1, size=(n, k)).astype(np.float32)
        got, tail = _product(guarded, t, w, m, k, x)
        want, _ = _product(plain, t, w, m, k, x)
        assert (tail == GUARD).all(), (t, m, n, "the product wrote past its output")
        assert np.array_equal(got, want), (t, m, n)
    blocks, bad = guarded.check_guards()
    assert blocks > 0 and bad == 0, guarded.L.b200q_last_error(guarded.h)


@pytest.mark.parametrize("t,n_tok", [(A.Q4_K, 1), (A.Q4_K, 6), (A.Q4_K, 300), (A.Q6_K, 300), (A.Q4_0, 70), (A.IQ4_XS, 260), (A.Q5_K, 260)])
def test_routed_products_leave_every_guard_untouched(ctxs, t, n_tok):
    guarded, _ = ctxs
    n_expert, n_used, m, k = 12, 3, 136, 1280
    rng = np.random.default_rng(n_tok)
    w = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    ids = np.stack([rng.permutation(n_expert)[:n_used] for _ in range(n_tok)]).astype(np.int32)
    x = rng.normal(0, 1, size=(n_tok, 1, k)).astype(np.float32)
    rb = w.shape[2]
    dw, dx, di = guarded.upload(w), guarded.upload(x), guarded.upload(ids)
    n_out = n_tok * n_used * m
    dy, _ = _guarded_out(guarded, n_out)
    W = A.Tensor.make(t, [k, m, n_expert, 1], [A.block_bytes(t), rb, rb * m, rb * m * n_expert], dw)
    I = A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * n_used, 4 * n_used * n_tok, 4 * n_used * n_tok], di)
    guarded.graph_begin()
    guarded.mul_mat_id(W, A.Tensor.f32(dx, [k, 1, n_tok]), I, A.Tensor.f32(dy, [m, n_used, n_tok]))
    raw = guarded.download(dy, (n_out + 64,), np.uint32)
    for p in (dw, dx, di, dy):
        guarded.free(p)
    assert (raw[n_out:] == GUARD).all()
    assert (raw[:n_out] != GUARD).all(), "an output element was never written"
    blocks, bad = guarded.check_guards()
    assert blocks > 0 and bad == 0, guarded.L.b200q_last_error(guarded.h)


def test_fused_block_leaves_every_guard_untouched(ctxs):
    guarded, _ = ctxs
    t, n_exp, n_used, d_model, d_ff, n_tok = A.Q4_K, 8, 2, 512, 256, 37
    gw = np.stack([make_weights(t, d_ff, d_model, 800 + e) for e in range(n_exp)])
    uw = np.stack([make_weights(t, d_ff, d_model, 900 + e) for e in range(n_exp)])
    dn = np.stack([make_weights(t, d_model, d_ff, 1000 + e) for e in range(n_exp)])
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, size=(n_tok, d_model)).astype(np.float32)
    logits = rng.normal(0, 1.5, size=(n_tok, n_exp)).astype(np.float32)
    held = []

    def w3(arr, k, m):
        dev = guarded.upload(arr)
        held.append(dev)
        rb = arr.shape[-1]
        return A.Tensor.make(t, [k, m, n_exp, 1], [A.block_bytes(t), rb, rb * m, rb * m * n_exp], dev)

    G, U, D = w3(gw, d_model, d_ff), w3(uw, d_model, d_ff), w3(dn, d_ff, d_model)
    dx, dl = guarded.upload(x), guarded.upload(logits)
    dy, _ = _guarded_out(guarded, n_tok * d_model)
    guarded.graph_begin()
    guarded.moe_ffn(G, U, D, A.Tensor.f32(dx, [d_model, n_tok]), A.Tensor.f32(dl, [n_exp, n_tok]), n_used, 6.103515625e-5,
                    float("inf"), A.Tensor.f32(dy, [d_model, n_tok]))
    raw = guarded.download(dy, (n_tok * d_model + 64,), np.uint32)
    for p in held + [dx, dl, dy]:
        guarded.free(p)
    assert (raw[n_tok * d_model:] == GUARD).all()
    blocks, bad = guarded.check_guards()
    assert blocks > 0 and bad == 0, guarded.L.b200q_last_error(guarded.h)


def test_guard_check_needs_the_switch(ctxs):
    _, plain = ctxs
    blocks, bad = A.binding.C.c_int(0), A.binding.C.c_int(0)
    assert plain.L.b200q_debug_check_guards(plain.h, A.binding.C.byref(blocks), A.binding.C.byref(bad)) == A.INVALID
