"""GPU parity of MUL_MAT_ID through the C ABI against the CPU oracle. Cases follow the
reference's op-suite list (marfrit/arcint contrib/llama.cpp/patches/0103-opencl-id-int8-sg8.patch
:633-650, 0104-...:414-416, 0000-09-moe-routing-gemm-tiles.patch:1043-1053): token counts on
both sides of the per-pair / routed switch, few and many experts, duplicate ids, ids through
an offset view, rows not a multiple of 8, broadcast (ne11 = 1) and per-slot (ne11 = n_used)
activations, 512 experts with 10 used."""
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


def run_id(ctx, t, w, m, k, x, ids_full, off, n_used):
    """w uint8 [n_expert, m, row_bytes]; x f32 [n_tok, ne11, k]; ids_full int32 [n_tok, width], the op
    reads columns off..off+n_used (an offset view when off > 0)."""
    n_expert, n_tok, ne11 = w.shape[0], x.shape[0], x.shape[1]
    rb = w.shape[2]
    dw, dx, di = ctx.upload(w), ctx.upload(x), ctx.upload(ids_full)
    dy = ctx.alloc(n_tok * n_used * m * 4)
    W = A.Tensor.make(t, [k, m, n_expert, 1], [A.block_bytes(t), rb, rb * m, rb * m * n_expert], dw)
    X = A.Tensor.f32(dx, [k, ne11, n_tok])
    width = ids_full.shape[1]
    I = A.Tensor.make(A.I32, [n_used, n_tok, 1, 1], [4, 4 * width, 4 * width * n_tok, 4 * width * n_tok], di + 4 * off)
    Y = A.Tensor.f32(dy, [m, n_used, n_tok])
    ctx.graph_begin()
    ctx.stats_reset()
    ctx.mul_mat_id(W, X, I, Y)
    got = ctx.download(dy, (n_tok, n_used, m), np.float32)
    st = ctx.stats()
    for p in (dw, dx, di, dy):
        ctx.free(p)
    return got, st


def check(ctx, t, n_expert, n_used, n_tok, m, k, ne11_is_one, seed, off=0, dup=False):
    rng = np.random.default_rng(seed)
    w = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    ids_full = np.stack([rng.permutation(n_expert)[:n_used + off] if n_expert >= n_used + off
                         else rng.integers(0, n_expert, n_used + off) for _ in range(n_tok)]).astype(np.int32)
    if dup:
        ids_full[:, off + 1:off + 3] = ids_full[:, off:off + 1]       # the same expert in several slots of a token
    ne11 = 1 if ne11_is_one else n_used
    x = rng.normal(0, 1, size=(n_tok, ne11, k)).astype(np.float32)
    got, st = run_id(ctx, t, w, m, k, x, ids_full, off, n_used)
    ids = ids_full[:, off:off + n_used]
    ref = O.mul_mat_id(t, w, m, k, x, ids, f64=True)
    assert np.isfinite(got).all()
    e = rel_err(got.reshape(-1, m), ref.reshape(-1, m))
    assert e < TOL, (t, n_expert, n_used, n_tok, m, k, e)
    return st


@pytest.mark.parametrize("t", [A.Q4_K, A.Q5_K, A.Q4_0, A.IQ4_XS, A.IQ4_NL, A.Q6_K, A.Q8_0])
@pytest.mark.parametrize("n_tok", [1, 2, 4, 5, 16, 33])
def test_mul_mat_id_types_and_token_counts(ctx, t, n_tok):
    st = check(ctx, t, n_expert=16, n_used=4, n_tok=n_tok, m=72, k=512, ne11_is_one=(n_tok % 2 == 1), seed=n_tok + t)
    launches = st.get("gemv_id", 0) + st.get("gemv_id_unaligned", 0)     # rows of 16-byte multiples or not
    if n_tok <= 4:
        assert st.get("moe_route", 0) == 0 and launches == 1           # per-pair path, no route
    else:
        assert st["moe_route"] == 1 and launches == 4                  # one launch per tile size class


@pytest.mark.parametrize("n_expert", [2, 16, 64, 184])
def test_mul_mat_id_expert_counts(ctx, n_expert):
    check(ctx, A.Q4_K, n_expert=n_expert, n_used=2, n_tok=300, m=77, k=256, ne11_is_one=False, seed=n_expert)


def test_mul_mat_id_duplicates_and_offset_view(ctx):
    check(ctx, A.Q4_K, n_expert=8, n_used=4, n_tok=33, m=64, k=512, ne11_is_one=True, seed=1, off=3, dup=True)
    check(ctx, A.Q4_0, n_expert=8, n_used=4, n_tok=3, m=64, k=512, ne11_is_one=False, seed=2, off=1, dup=True)


@pytest.mark.parametrize("n_tok,ne11_is_one", [(1, True), (3, False), (64, True), (64, False)])
def test_mul_mat_id_512_experts_top10(ctx, n_tok, ne11_is_one):
    """benchmark config 5's shapes: 512 experts, top-10, gate/up 512 x 2048 and down 2048 x 512 (fewer rows here)."""
    rng = np.random.default_rng(7)
    t, n_expert, n_used, m, k = A.Q4_K, 512, 10, 64, 2048
    base = [O.random_blocks(t, m, k, rng) for _ in range(8)]
    w = np.stack([base[e % 8] for e in range(n_expert)])
    w[:, :, 0] = (np.arange(n_expert) % 251)[:, None]                 # experts differ in their first scale byte
    ids = O.route_ids(n_used, n_tok, n_expert, 99)
    x = rng.normal(0, 1, size=(n_tok, 1 if ne11_is_one else n_used, k)).astype(np.float32)
    got, st = run_id(ctx, t, w, m, k, x, ids, 0, n_used)
    ref = O.mul_mat_id(t, w, m, k, x, ids, f64=True)
    assert rel_err(got.reshape(-1, m), ref.reshape(-1, m)) < TOL


def test_route_is_shared_within_a_graph(ctx):
    """gate, up and down of a layer use one route (the reference's route cache)."""
    t, n_expert, n_used, n_tok, m, k = A.Q4_K, 32, 4, 40, 64, 256
    rng = np.random.default_rng(3)
    w = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    ids = rng.integers(0, n_expert, size=(n_tok, n_used)).astype(np.int32)
    x = rng.normal(0, 1, size=(n_tok, 1, k)).astype(np.float32)
    rb = w.shape[2]
    dw, dx, di, dy = ctx.upload(w), ctx.upload(x), ctx.upload(ids), ctx.alloc(n_tok * n_used * m * 4)
    W = A.Tensor.make(t, [k, m, n_expert, 1], [144, rb, rb * m, rb * m * n_expert], dw)
    X, I, Y = A.Tensor.f32(dx, [k, 1, n_tok]), A.Tensor.make(A.I32, [n_used, n_tok], [4, 4 * n_used], di), A.Tensor.f32(dy, [m, n_used, n_tok])
    ctx.graph_begin()
    ctx.stats_reset()
    for _ in range(3):
        ctx.mul_mat_id(W, X, I, Y)
    st = ctx.stats()
    assert st["moe_route"] == 1 and st["route_cache_hit"] == 2 and st["quantize_act_q8_256"] == 1
    ctx.graph_begin()
    ctx.mul_mat_id(W, X, I, Y)
    assert ctx.stats()["moe_route"] == 2
    for p in (dw, dx, di, dy):
        ctx.free(p)


def test_mul_mat_id_shape_errors(ctx):
    d = ctx.alloc(4096)
    W = A.Tensor.make(A.Q4_K, [256, 8, 4, 1], [144, 144, 144 * 8, 144 * 32], d)
    I = A.Tensor.make(A.I32, [2, 3], [4, 8], d)
    Y = A.Tensor.f32(d, [8, 2, 3])
    assert ctx.L.b200q_mul_mat_id(ctx.h, W, A.Tensor.f32(d, [256, 3, 3]), I, Y) == A.INVALID      # ne11 not 1 or n_used
    assert ctx.L.b200q_mul_mat_id(ctx.h, W, A.Tensor.f32(d, [256, 1, 3]), A.Tensor.make(A.F32, [2, 3], [4, 8], d), Y) == A.UNSUPPORTED
    assert ctx.L.b200q_mul_mat_id(ctx.h, W, A.Tensor.f32(d, [256, 1, 3]), I, A.Tensor.f32(d, [8, 3, 3])) == A.INVALID
    assert ctx.supports(A.OP_MUL_MAT_ID, W, A.Tensor.f32(d, [256, 1, 3]), I, Y) == A.OK
    ctx.free(d)


# ---- prompt-sized batches: the route's 128-pair tiles through the tensor-core GEMM ----

@pytest.mark.parametrize("t", [A.Q4_K, A.Q5_K, A.IQ4_XS, A.IQ4_NL, A.Q4_0, A.Q8_0])
@pytest.mark.parametrize("n_expert,n_used,n_tok,ne11_is_one", [(8, 2, 300, True), (8, 2, 300, False), (4, 4, 700, True),
                                                               (32, 8, 64, False)])
def test_mul_mat_id_tensor_core_tiles(ctx, t, n_expert, n_used, n_tok, ne11_is_one):
    st = check(ctx, t, n_expert=n_expert, n_used=n_used, n_tok=n_tok, m=200, k=1024, ne11_is_one=ne11_is_one,
               seed=n_tok + n_expert)
    assert st.get("moe_gemm", 0) == 1 and st.get("gemm_tc", 0) == 1, st
    assert st.get("gemv_id", 0) + st.get("gemv_id_unaligned", 0) == 0


def test_mul_mat_id_tensor_core_skewed_route_duplicates_offset(ctx):
    """Zipf-skewed routing (some experts with hundreds of pairs, some with none), the same expert in
    several slots of a token, ids read through an offset view."""
    t, n_expert, n_used, n_tok, m, k = A.Q4_K, 16, 4, 400, 136, 512
    rng = np.random.default_rng(11)
    w = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    ids_full = np.concatenate([rng.integers(0, n_expert, (n_tok, 2)).astype(np.int32),
                               O.route_ids(n_used, n_tok, n_expert, 5, 2.0)], axis=1)
    ids_full[::3, 3] = ids_full[::3, 2]
    ids_full[:, :][ids_full == 7] = 6                                     # expert 7 gets nothing
    x = rng.normal(0, 1, size=(n_tok, n_used, k)).astype(np.float32)
    got, st = run_id(ctx, t, w, m, k, x, ids_full, 2, n_used)
    assert st.get("moe_gemm", 0) == 1
    ref = O.mul_mat_id(t, w, m, k, x, ids_full[:, 2:2 + n_used], f64=True)
    assert rel_err(got.reshape(-1, m), ref.reshape(-1, m)) < TOL


def test_config5_moe_q4_K_prompt_batch(ctx):
    """benchmark config 5 at a prompt batch: 512 experts, top-10, 2048 tokens, gate shape 512 x 2048;
    sampled tokens against the oracle."""
    t, n_expert, n_used, n_tok, m, k = A.Q4_K, 512, 10, 2048, 512, 2048
    rng = np.random.default_rng(12)
    base = [O.random_blocks(t, m, k, rng) for _ in range(4)]
    w = np.stack([base[e % 4] for e in range(n_expert)])
    w[:, :, 0] = (np.arange(n_expert) % 251)[:, None]
    ids = O.route_ids(n_used, n_tok, n_expert, 0x5EED0800)
    x = O.fill_normal(n_tok * k, 13, 1.0).reshape(n_tok, 1, k)
    got, st = run_id(ctx, t, w, m, k, x, ids, 0, n_used)
    assert st.get("moe_gemm", 0) == 1
    ts = np.arange(0, n_tok, 97)
    ref = O.mul_mat_id(t, w, m, k, x[ts], np.ascontiguousarray(ids[ts]), f64=True)
    assert rel_err(got[ts].reshape(-1, m), ref.reshape(-1, m)) < TOL
    assert np.isfinite(got).all()


def test_mul_mat_id_tensor_core_q6_K(ctx):
    st = check(ctx, A.Q6_K, n_expert=8, n_used=2, n_tok=300, m=200, k=2048, ne11_is_one=True, seed=77)
    assert st.get("moe_gemm", 0) == 1 and st.get("gemm_tc", 0) == 1, st


def test_mul_mat_id_tensor_core_q6_K_rows_not_16_byte_multiples(ctx):
    """Five super-blocks per row (1050 bytes): the experts' rows are staged one by one, each at its own offset."""
    st = check(ctx, A.Q6_K, n_expert=8, n_used=2, n_tok=300, m=200, k=1280, ne11_is_one=True, seed=78)
    assert st.get("moe_gemm", 0) == 1 and st.get("gemm_tc", 0) == 1 and st.get("gemm_kq_rowcopy", 0) == 1, st


def test_mul_mat_id_tensor_core_iq4_xs_odd_superblock_count(ctx):
    st = check(ctx, A.IQ4_XS, n_expert=8, n_used=2, n_tok=300, m=200, k=768, ne11_is_one=True, seed=79)
    assert st.get("moe_gemm", 0) == 1 and st.get("gemm_tc", 0) == 1 and st.get("gemm_kq_rowcopy", 0) == 1, st


def test_gate_and_up_share_the_gathered_activation(ctx):
    """Two MUL_MAT_ID calls of one graph over the same src1 and ids (gate and up of a layer) gather and quantize the
    activation once; a third with another src1 (down) does it again; results stay right."""
    t, n_expert, n_used, n_tok, m, k = A.Q4_K, 8, 2, 300, 136, 512
    rng = np.random.default_rng(21)
    w1 = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    w2 = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    ids = rng.integers(0, n_expert, size=(n_tok, n_used)).astype(np.int32)
    x = rng.normal(0, 1, size=(n_tok, 1, k)).astype(np.float32)
    x2 = rng.normal(0, 1, size=(n_tok, n_used, k)).astype(np.float32)
    rb = w1.shape[2]
    d1, d2, dx, dx2, di = ctx.upload(w1), ctx.upload(w2), ctx.upload(x), ctx.upload(x2), ctx.upload(ids)
    y1, y2, y3 = (ctx.alloc(n_tok * n_used * m * 4) for _ in range(3))
    W = lambda d: A.Tensor.make(t, [k, m, n_expert, 1], [144, rb, rb * m, rb * m * n_expert], d)
    I = A.Tensor.make(A.I32, [n_used, n_tok], [4, 4 * n_used], di)
    Y = lambda d: A.Tensor.f32(d, [m, n_used, n_tok])
    ctx.graph_begin()
    ctx.stats_reset()
    ctx.mul_mat_id(W(d1), A.Tensor.f32(dx, [k, 1, n_tok]), I, Y(y1))
    ctx.mul_mat_id(W(d2), A.Tensor.f32(dx, [k, 1, n_tok]), I, Y(y2))
    ctx.mul_mat_id(W(d1), A.Tensor.f32(dx2, [k, n_used, n_tok]), I, Y(y3))
    st = ctx.stats()
    assert st["moe_gemm"] == 3 and st["gemm_tc_quantize"] == 2 and st["moe_route"] == 1, st
    for dy, w, xx in ((y1, w1, x), (y2, w2, x), (y3, w1, x2)):
        got = ctx.download(dy, (n_tok, n_used, m), np.float32)
        ref = O.mul_mat_id(t, w, m, k, xx, ids, f64=True)
        assert rel_err(got.reshape(-1, m), ref.reshape(-1, m)) < TOL
    for p in (d1, d2, dx, dx2, di, y1, y2, y3):
        ctx.free(p)
