"""The MoE router and the fused feed-forward block through the C ABI against the oracle.

The router restates the reference's kernel_topk_moe_softmax_norm_n* (marfrit/arcint contrib/llama.cpp/patches/
0000-09-moe-routing-gemm-tiles.patch:928-987): ids must match exactly (ties go to the lower expert), weights
to float rounding. The block is checked against the fp64 chain on the same quantized operands with the
reference op suite's NMSE bound (the intermediate h is re-quantized for the down projection, so a last-bit
difference in h can move an int8 code), and against the library's own unfused sequence."""
import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from gpu_util import make_weights, nmse, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = A.Context(0)
    yield c
    c.close()


def run_router(ctx, logits, n_used, cmin, cmax):
    n_tok, n_exp = logits.shape
    dl, di, dw = ctx.upload(logits), ctx.alloc(n_tok * n_used * 4), ctx.alloc(n_tok * n_used * 4)
    ctx.moe_router(A.Tensor.f32(dl, [n_exp, n_tok]), n_used, cmin, cmax,
                   A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * n_used], di), A.Tensor.f32(dw, [n_used, n_tok]))
    ids, w = ctx.download(di, (n_tok, n_used), np.int32), ctx.download(dw, (n_tok, n_used), np.float32)
    for p in (dl, di, dw):
        ctx.free(p)
    return ids, w


@pytest.mark.parametrize("n_exp,n_used,n_tok", [(8, 2, 5), (60, 4, 33), (128, 8, 7), (512, 10, 300), (1000, 32, 3)])
def test_router_matches_the_reference_rule(ctx, n_exp, n_used, n_tok):
    rng = np.random.default_rng(n_exp + n_used)
    logits = rng.normal(0, 2, size=(n_tok, n_exp)).astype(np.float32)
    logits[0, :] = 0.25                                    # a row of ties: experts 0, 1, 2, ... in order
    if n_exp > 40:
        logits[1, 7] = logits[1, 33] = logits[1].max() + 1.0      # a tie for first place: 7 before 33
    for cmin, cmax in ((6.103515625e-5, np.inf), (0.9, 1.1)):
        ids, w = run_router(ctx, logits, n_used, cmin, cmax)
        want_ids, want_w = O.moe_router(logits, n_used, cmin, cmax)
        assert np.array_equal(ids, want_ids)
        assert np.allclose(w, want_w, rtol=2e-6, atol=1e-9)
        assert list(ids[0]) == list(range(n_used))


def test_router_limits(ctx):
    d = ctx.alloc(1 << 16)
    L = ctx.L
    big = A.Tensor.f32(d, [2000, 1])
    assert L.b200q_moe_router(ctx.h, big, 2, 0.0, 1.0, A.Tensor.make(A.I32, [2, 1, 1, 1], [4, 8], d), A.Tensor.f32(d, [2, 1])) == A.UNSUPPORTED
    assert b"experts" in L.b200q_last_error(ctx.h)
    ctx.free(d)


@pytest.mark.parametrize("t,n_exp,n_used,d_model,d_ff,n_tok", [(A.Q4_K, 8, 2, 512, 256, 3), (A.Q4_K, 16, 4, 512, 256, 200),
                                                               (A.Q4_0, 8, 2, 256, 128, 64), (A.IQ4_XS, 8, 3, 512, 512, 150)])
def test_ffn_block_against_the_fp64_chain_and_the_unfused_sequence(ctx, t, n_exp, n_used, d_model, d_ff, n_tok):
    gw = np.stack([make_weights(t, d_ff, d_model, 800 + e) for e in range(n_exp)])
    uw = np.stack([make_weights(t, d_ff, d_model, 900 + e) for e in range(n_exp)])
    dw_ = np.stack([make_weights(t, d_model, d_ff, 1000 + e) for e in range(n_exp)])
    rng = np.random.default_rng(n_tok)
    x = rng.normal(0, 1, size=(n_tok, d_model)).astype(np.float32)
    logits = rng.normal(0, 1.5, size=(n_tok, n_exp)).astype(np.float32)
    cmin, cmax = 6.103515625e-5, float("inf")
    want, want_ids, want_w = O.moe_ffn(t, gw, uw, dw_, d_model, d_ff, x, logits, n_used, cmin, cmax)

    def w3(arr, k, m):
        dev = ctx.upload(arr)
        rb = arr.shape[-1]
        return dev, A.Tensor.make(t, [k, m, n_exp, 1], [A.block_bytes(t), rb, rb * m, rb * m * n_exp], dev)

    dg, G = w3(gw, d_model, d_ff)
    du, U = w3(uw, d_model, d_ff)
    dd, D = w3(dw_, d_ff, d_model)
    dx, dl, dy = ctx.upload(x), ctx.upload(logits), ctx.alloc(n_tok * d_model * 4)
    di, dwt = ctx.alloc(n_tok * n_used * 4), ctx.alloc(n_tok * n_used * 4)
    I = A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * n_used], di)
    Wt = A.Tensor.f32(dwt, [n_used, n_tok])
    ctx.graph_begin()
    ctx.stats_reset()
    ctx.moe_ffn(G, U, D, A.Tensor.f32(dx, [d_model, n_tok]), A.Tensor.f32(dl, [n_exp, n_tok]), n_used, cmin, cmax,
                A.Tensor.f32(dy, [d_model, n_tok]), I, Wt)
    got = ctx.download(dy, (n_tok, d_model), np.float32)
    st = ctx.stats()
    assert st.get("moe_ffn") == 1 and st.get("moe_router") == 1
    assert np.array_equal(ctx.download(di, (n_tok, n_used), np.int32), want_ids)
    assert np.isfinite(got).all()
    assert nmse(got, want) < 5e-4, nmse(got, want)
    # the unfused sequence through the same entry points: identical arithmetic, so equal up to nothing
    dgo, duo, ddo = ctx.alloc(n_tok * n_used * d_ff * 4), ctx.alloc(n_tok * n_used * d_ff * 4), ctx.alloc(n_tok * n_used * d_model * 4)
    ctx.graph_begin()
    X3 = A.Tensor.f32(dx, [d_model, 1, n_tok])
    ctx.mul_mat_id(G, X3, I, A.Tensor.f32(dgo, [d_ff, n_used, n_tok]))
    ctx.mul_mat_id(U, X3, I, A.Tensor.f32(duo, [d_ff, n_used, n_tok]))
    g = ctx.download(dgo, (n_tok, n_used, d_ff), np.float32)
    u = ctx.download(duo, (n_tok, n_used, d_ff), np.float32)
    h = (g.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64))) * u).astype(np.float32)
    dh = ctx.upload(h)
    ctx.graph_begin()
    ctx.mul_mat_id(D, A.Tensor.f32(dh, [d_ff, n_used, n_tok]), I, A.Tensor.f32(ddo, [d_model, n_used, n_tok]))
    dn = ctx.download(ddo, (n_tok, n_used, d_model), np.float32)
    wt = ctx.download(dwt, (n_tok, n_used), np.float32)
    seq = (dn.astype(np.float64) * wt[:, :, None]).sum(axis=1)
    assert nmse(got, seq) < 1e-6, nmse(got, seq)
    for p in (dg, du, dd, dx, dl, dy, di, dwt, dgo, duo, ddo, dh):
        ctx.free(p)
