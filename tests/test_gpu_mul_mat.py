"""GPU parity of MUL_MAT through the C ABI against the CPU oracle.

Bars: decoded weights and quantized activations bit-exact; f32 outputs within max relative
error 1e-3 of the fp64 product of the same quantized operands (TOL in gpu_util). Shapes
follow the reference's op-suite cases (marfrit/arcint contrib/llama.cpp/patches/
0000-01-kquant-integer-dpas.patch:3965-4035, 0115-...-few-column-...patch:1057-1085)."""
import numpy as np
import pytest

import arcint_b200 as A
import oracle as O
from gpu_util import TOL, make_weights, nmse, rel_err

pytestmark = pytest.mark.gpu

TYPES = [A.Q4_0, A.Q8_0, A.Q4_K, A.Q5_K, A.Q6_K, A.IQ4_XS, A.IQ4_NL]
NAMES = {A.Q4_0: "q4_0", A.Q8_0: "q8_0", A.Q4_K: "q4_K", A.Q5_K: "q5_K", A.Q6_K: "q6_K", A.IQ4_XS: "iq4_xs", A.IQ4_NL: "iq4_nl"}


@pytest.fixture(scope="module")
def ctx():
    c = A.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("t", TYPES)
def test_device_decode_bit_exact(ctx, golden, t):
    blocks, want = golden[NAMES[t] + "_blocks"], golden[NAMES[t] + "_deq"]
    m, k = want.shape
    dw, do = ctx.upload(blocks), ctx.alloc(want.nbytes)
    ctx.check(ctx.L.b200q_debug_dequantize(ctx.h, A.Tensor.weights(t, dw, k, m), do))
    got = ctx.download(do, want.shape, np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ctx.free(dw), ctx.free(do)


def _device_quantize(ctx, t, x):
    n, k = x.shape
    dx = ctx.upload(x)
    dq, ds, db = ctx.alloc(n * k), ctx.alloc(n * (k // 32) * 4), ctx.alloc(n * (k // 32) * 2)
    ctx.check(ctx.L.b200q_debug_quantize_act(ctx.h, t, A.Tensor.f32(dx, [k, n]), dq, ds, db))
    q = ctx.download(dq, (n, k), np.int8)
    if O.act_form(t) == O.ACT_Q8_0:
        d = ctx.download(ds, (n, k // 32), np.uint16)
        s = None
    else:
        d = ctx.download(ds, (n, k // 256), np.float32)
        s = ctx.download(db, (n, k // 32), np.int16)
    for p in (dx, dq, ds, db):
        ctx.free(p)
    return q, d, s


def test_activation_q8_0_bit_exact_golden(ctx, golden):
    q, d, _ = _device_quantize(ctx, A.Q4_0, golden["act_src"])
    assert np.array_equal(q, golden["act_q"]) and np.array_equal(d, golden["act_d"])


def test_activation_quantizers_bit_exact_oracle(ctx):
    x = O.fill_normal(16 * 4096, 21, 1.0).reshape(16, 4096)
    x[3, :512] = 0.0
    x[4, 256:512] = 1e-35
    x[5] = np.round(x[5] * 2) / 2                        # exact .5 ties
    q, d, _ = _device_quantize(ctx, A.Q8_0, x)
    oq, od = O.quantize_act_q8_0(x)
    assert np.array_equal(q, oq) and np.array_equal(d, od)
    q, d, s = _device_quantize(ctx, A.Q4_K, x)
    oq, od, os_ = O.quantize_act_q8_256(x)
    assert np.array_equal(q, oq) and np.array_equal(d.view(np.uint32), od.view(np.uint32)) and np.array_equal(s, os_)


SHAPES_32 = [(256, 2560), (1001, 2560), (77, 4096), (512, 14336), (300, 1024), (64, 2080), (33, 96), (1, 32)]
SHAPES_256 = [(256, 2560), (1001, 2560), (77, 4096), (512, 14336), (300, 1024), (1023, 4096), (5, 256), (64, 2816)]


def _check(ctx, t, w, k, x, tol=TOL):
    got = ctx.run_mul_mat(t, w, k, x)
    ref = O.mul_mat_f64(t, w, k, x, True)
    assert np.isfinite(got).all()
    e = rel_err(got, ref)
    assert e < tol, (NAMES[t], w.shape, x.shape, e)
    return got


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 6, 7, 8])
def test_decode_widths(ctx, t, n):
    rng = np.random.default_rng(17 * t + n)
    for m, k in (SHAPES_32 if A.block_size(t) == 32 else SHAPES_256):
        w = O.random_blocks(t, m, k, rng)
        x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
        _check(ctx, t, w, k, x)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n", [9, 12, 16, 17, 40, 64, 100])
def test_wider_products(ctx, t, n):
    rng = np.random.default_rng(31 * t + n)
    for m, k in [(300, 1024), (256, 2560)]:
        w = make_weights(t, m, k, 900 + t)
        x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
        got = _check(ctx, t, w, k, x)
        # the reference's op-suite bound against the unquantized-activation product
        assert nmse(got, O.mul_mat_f64(t, w, k, x, False)) < 5e-4


def test_red_case_wrong_scale_is_caught(ctx):
    """A test must be able to fail: results for a perturbed input must NOT pass the bar."""
    t, m, k = A.Q4_K, 64, 1024
    rng = np.random.default_rng(2)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(2, k)).astype(np.float32)
    ref = O.mul_mat_f64(t, w, k, x, True)
    x[1, 300] += 1.0
    assert rel_err(ctx.run_mul_mat(t, w, k, x), ref) > TOL


def test_weight_broadcast_over_src1_dims(ctx):
    """nr = {2,1}: the weight is broadcast over src1's dimension 2, flattened into columns."""
    t, m, k, n = A.Q4_K, 96, 1024, 3
    rng = np.random.default_rng(3)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(2, n, k)).astype(np.float32)          # [ne2][ne1][K]
    dw, dx, dy = ctx.upload(w), ctx.upload(x), ctx.alloc(2 * n * m * 4)
    ctx.graph_begin()
    ctx.mul_mat(A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dx, [k, n, 2]), A.Tensor.f32(dy, [m, n, 2]))
    got = ctx.download(dy, (2 * n, m), np.float32)
    assert rel_err(got, O.mul_mat_f64(t, w, k, x.reshape(2 * n, k), True)) < TOL
    for p in (dw, dx, dy):
        ctx.free(p)


def test_permuted_src1(ctx):
    """per = {0,2,1,3}: src1 is [K, 1, n] in shape with a column stride that is not nb[1]."""
    t, m, k, n = A.Q8_0, 64, 256, 5
    rng = np.random.default_rng(4)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    dw, dx, dy = ctx.upload(w), ctx.upload(x), ctx.alloc(n * m * 4)
    src1 = A.Tensor.make(A.F32, [k, 1, n, 1], [4, 4 * k * n, 4 * k, 4 * k * n], dx)
    dst = A.Tensor.make(A.F32, [m, 1, n, 1], [4, 4 * m * n, 4 * m, 4 * m * n], dy)
    ctx.graph_begin()
    ctx.mul_mat(A.Tensor.weights(t, dw, k, m), src1, dst)
    got = ctx.download(dy, (n, m), np.float32)
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL
    for p in (dw, dx, dy):
        ctx.free(p)


def test_padded_dst_and_row_stride(ctx):
    """dst columns further apart than M; weight rows further apart than their bytes."""
    t, m, k, n = A.Q4_0, 50, 512, 4
    rng = np.random.default_rng(6)
    w = O.random_blocks(t, m, k, rng)
    rb = w.shape[1]
    wp = np.zeros((m, rb + 14), dtype=np.uint8)                      # stride 302: not a multiple of 16
    wp[:, :rb] = w
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    dw, dx, dy = ctx.upload(wp), ctx.upload(x), ctx.alloc(n * (m + 6) * 4)
    src0 = A.Tensor.make(t, [k, m, 1, 1], [18, rb + 14, (rb + 14) * m, (rb + 14) * m], dw)
    dst = A.Tensor.make(A.F32, [m, n, 1, 1], [4, 4 * (m + 6), 4 * (m + 6) * n, 4 * (m + 6) * n], dy)
    ctx.graph_begin()
    ctx.mul_mat(src0, A.Tensor.f32(dx, [k, n]), dst)
    got = ctx.download(dy, (n, m + 6), np.float32)[:, :m]
    assert rel_err(got, O.mul_mat_f64(t, w, k, x, True)) < TOL
    for p in (dw, dx, dy):
        ctx.free(p)


def test_empty_and_unsupported(ctx):
    t, k = A.Q4_K, 512
    dw = ctx.alloc(1024)
    w0 = A.Tensor.weights(t, dw, k, 0)
    assert ctx.mul_mat_status(w0, A.Tensor.f32(dw, [k, 3]), A.Tensor.f32(dw, [0, 3])) == A.OK     # no rows
    w1 = A.Tensor.weights(t, dw, k, 2)
    assert ctx.mul_mat_status(w1, A.Tensor.f32(dw, [k, 0]), A.Tensor.f32(dw, [2, 0])) == A.OK     # no columns
    assert ctx.mul_mat_status(A.Tensor.weights(t, dw, 300, 2), A.Tensor.f32(dw, [300, 1]),
                              A.Tensor.f32(dw, [2, 1])) == A.UNSUPPORTED                         # K % 256
    assert ctx.mul_mat_status(A.Tensor.weights(t, dw, k, 2, 3), A.Tensor.f32(dw, [k, 1]),
                              A.Tensor.f32(dw, [2, 1])) == A.UNSUPPORTED                         # 3-D weights
    assert b"3-D" in ctx.L.b200q_last_error(ctx.h)
    ctx.free(dw)


def test_activation_cache_within_a_graph(ctx):
    """q/k/v share one quantized activation inside a graph; a new graph re-quantizes."""
    t, m, k = A.Q4_0, 64, 1024
    rng = np.random.default_rng(8)
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(3, k)).astype(np.float32)      # three columns: not the width that quantizes inside the GEMV
    dw, dx, dy = ctx.upload(w), ctx.upload(x), ctx.alloc(3 * m * 4)
    W, X, Y = A.Tensor.weights(t, dw, k, m), A.Tensor.f32(dx, [k, 3]), A.Tensor.f32(dy, [m, 3])
    ctx.stats_reset()
    ctx.graph_begin()
    for _ in range(3):
        ctx.mul_mat(W, X, Y)
    s = ctx.stats()
    assert s["quantize_act_q8_0"] == 1 and s["act_cache_hit"] == 2 and s["gemv_3col"] == 3
    x2 = x * 2
    ctx.upload(x2, dx)
    ctx.graph_begin()
    ctx.mul_mat(W, X, Y)
    assert ctx.stats()["quantize_act_q8_0"] == 2
    assert rel_err(ctx.download(dy, (3, m), np.float32), O.mul_mat_f64(t, w, k, x2, True)) < TOL
    for p in (dw, dx, dy):
        ctx.free(p)


@pytest.mark.parametrize("t,m,k", [(A.Q4_K, 11008, 4096), (A.Q4_K, 4096, 11008), (A.Q6_K, 32000, 4096),
                                   (A.Q4_0, 4096, 4096), (A.Q8_0, 3072, 3072), (A.IQ4_XS, 5120, 17408)])
def test_full_size_decode_shapes_sampled_rows(ctx, t, m, k):
    """The benchmark's decode shapes at batch 1 and 8: every output is produced, sampled rows are
    checked against the oracle (rows are independent, so a row subset is a valid oracle case)."""
    rng = np.random.default_rng(m + k)
    base = make_weights(t, 512, k, 40 + t)
    w = np.tile(base, (-(-m // 512), 1))[:m].copy()
    w[:, :2] = w[rng.permutation(m), :2]                             # rows differ in their first scale
    x = rng.normal(0, 1, size=(8, k)).astype(np.float32)
    rows = np.unique(np.concatenate([[0, 1, m - 2, m - 1], rng.integers(0, m, 60)]))
    for n in (1, 8):
        got = ctx.run_mul_mat(t, w, k, x[:n])
        assert np.isfinite(got).all()
        ref = O.mul_mat_f64(t, w[rows], k, x[:n], True)
        sub = got[:, rows]
        floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
        assert float((np.abs(sub - ref) / np.maximum(np.abs(ref), floor)).max()) < TOL


def test_overlapped_host_copies_eager_and_in_a_graph(ctx):
    """b200q_tensor_stage / _fetch (uploads and downloads on the context's copy streams) around a chain of
    products, each with its own buffers: the host results equal the plain upload / download path, called
    eagerly and replayed as a CUDA graph with new inputs."""
    t, m, k = A.Q4_K, 640, 1024
    w = make_weights(t, m, k, 90)
    dw = ctx.upload(w)
    widths = [1, 3, 8, 5]
    hin = [A.binding.PinnedArray((n, k), np.float32) for n in widths]
    hout = [A.binding.PinnedArray((n, m), np.float32) for n in widths]
    din = [ctx.alloc(4 * n * k) for n in widths]
    dout = [ctx.alloc(4 * n * m) for n in widths]

    def fill(seed):
        for i, n in enumerate(widths):
            hin[i].array[:] = O.fill_normal(n * k, seed + i, 1.0).reshape(n, k)
            hout[i].array[:] = 0

    def chain():
        for i, n in enumerate(widths):
            ctx.graph_begin()
            ctx.stage(din[i], hin[i].ptr, 4 * n * k)
            ctx.mul_mat(A.Tensor.weights(t, dw, k, m), A.Tensor.f32(din[i], [k, n]), A.Tensor.f32(dout[i], [m, n]))
            ctx.fetch(hout[i].ptr, dout[i], 4 * n * m)

    def check():
        for i, n in enumerate(widths):
            want = ctx.run_mul_mat(t, w, k, np.array(hin[i].array))
            assert np.array_equal(hout[i].array, want), (i, n)

    fill(100)
    chain()
    ctx.sync()
    check()
    g = ctx.capture(chain)
    fill(200)
    ctx.graph_launch(g)
    ctx.sync()
    check()
    ctx.graph_free(g)
    for p in din + dout + [dw]:
        ctx.free(p)
    for h in hin + hout:
        h.free()


@pytest.mark.parametrize("t", [A.Q4_0, A.Q8_0])
@pytest.mark.parametrize("m,k,n", [(512, 4096, 1), (96, 2304, 2), (1000, 512, 1), (37, 256, 2)])
def test_gemv_that_quantizes_its_own_activation_is_bit_identical(t, m, k, n):
    """With B200Q_FUSE_QUANT_BYTES set, small per-32 decode products quantize their slice of the activation inside the
    GEMV (one launch instead of two; off by default). The arithmetic is the quantizer kernel's, operation for
    operation, so the result must equal the two-kernel route bit for bit."""
    import os
    w = make_weights(t, m, k, 60 + t)
    x = np.random.default_rng(m + k).normal(0, 1, size=(n, k)).astype(np.float32)
    x[0, :32] = 0.0                                        # an all-zero block: scale 0, codes 0
    outs = {}
    for fused in (True, False):
        os.environ["B200Q_FUSE_QUANT_BYTES"] = str(4 << 20) if fused else "0"
        os.environ["B200Q_GEMV_STREAM_MASK"] = "0x1FE"          # the same GEMV kernel at every width, so only the quantizer's place differs
        try:
            with A.Context(0) as c:
                outs[fused] = c.run_mul_mat(t, w, k, x)
                assert (c.stats().get("gemv_fused_quant", 0) == 1) == fused, c.stats()
        finally:
            os.environ.pop("B200Q_FUSE_QUANT_BYTES", None)
            os.environ.pop("B200Q_GEMV_STREAM_MASK", None)
    assert np.array_equal(outs[True], outs[False])
    assert rel_err(outs[True], O.mul_mat_f64(t, w, k, x, True)) < TOL
