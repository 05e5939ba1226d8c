"""The CPU oracle against its pins: gguf-py golden vectors (committed), the
reference's own kq_i8_ops.inc (when it was built from the reference tree), and the
device-free checks the reference's tests make on this path
(0000-09-moe-routing-gemm-tiles.patch:1095-1697: exact decode of random blocks,
.5-away rounding at scale 1, the amax/127 scale, the MUL_MAT_ID column rule)."""
import numpy as np
import pytest

import oracle as O

NAMES = {"q4_0": O.Q4_0, "q8_0": O.Q8_0, "q4_K": O.Q4_K, "q5_K": O.Q5_K, "q6_K": O.Q6_K, "iq4_xs": O.IQ4_XS, "iq4_nl": O.IQ4_NL}
SIZES = {O.Q4_0: (32, 18), O.Q8_0: (32, 34), O.Q4_K: (256, 144), O.Q5_K: (256, 176), O.Q6_K: (256, 210), O.IQ4_XS: (256, 136), O.IQ4_NL: (32, 18)}


def test_block_sizes():
    for t, (bs, bb) in SIZES.items():
        assert O.block_size(t) == bs and O.block_bytes(t) == bb
        assert O.row_bytes(t, 4096) == 4096 // bs * bb


def test_fp16_roundtrip_all_values():
    L = O.lib()
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([L.orc_fp16_to_fp32(int(v)) for v in h], dtype=np.float32)
    fin = np.isfinite(want)
    assert np.array_equal(got[fin], want[fin])
    back = np.array([L.orc_fp32_to_fp16(float(v)) for v in want[fin]], dtype=np.uint16)
    assert np.array_equal(back, h[fin])


def test_fp32_to_fp16_rounding_matches_numpy():
    rng = np.random.default_rng(1)
    v = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 2000), rng.normal(0, 3e4, 2000),
                        [65504.0, 65519.9, 65520.0, 1e-8, 6e-8, 2.98e-8, 2.99e-8]]).astype(np.float32)
    L = O.lib()
    got = np.array([L.orc_fp32_to_fp16(float(x)) for x in v], dtype=np.uint16)
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("name", list(NAMES))
def test_dequantize_matches_gguf_golden(golden, name):
    t = NAMES[name]
    blocks, want = golden[name + "_blocks"], golden[name + "_deq"]
    got = O.dequantize(t, blocks, want.shape[1])
    assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequantize_red_case(golden):
    """A test must be able to fail: one flipped code bit has to show."""
    blocks = golden["q4_0_blocks"].copy()
    blocks[0, 2] ^= 0x01
    got = O.dequantize(O.Q4_0, blocks, golden["q4_0_deq"].shape[1])
    assert not np.array_equal(got, golden["q4_0_deq"])


@pytest.mark.parametrize("name", ["q4_0", "q8_0"])
def test_quantize_matches_gguf_golden(golden, name):
    got = O.quantize(NAMES[name], golden[name + "_src"])
    assert np.array_equal(got, golden[name + "_quant"])


def test_act_q8_0_matches_gguf_golden(golden):
    q, d = O.quantize_act_q8_0(golden["act_src"])
    assert np.array_equal(q, golden["act_q"]) and np.array_equal(d, golden["act_d"])


@pytest.mark.parametrize("t", [O.Q4_K, O.Q5_K, O.Q6_K, O.IQ4_XS, O.IQ4_NL, O.Q4_0, O.Q8_0])
def test_standin_quantizers_are_close(t):
    """The stand-in quantizers must produce valid blocks whose decode is near the input."""
    w = O.fill_normal(8 * 1024, 7, 0.02).reshape(8, 1024)
    deq = O.dequantize(t, O.quantize(t, w), 1024)
    rel = np.sqrt(np.mean((deq - w) ** 2)) / np.sqrt(np.mean(w ** 2))
    assert rel < {O.Q4_0: 0.12, O.Q8_0: 0.01, O.Q4_K: 0.09, O.Q5_K: 0.05, O.Q6_K: 0.03, O.IQ4_XS: 0.09, O.IQ4_NL: 0.09}[t]


def test_act_q8_256_rule():
    """kernel_quant_i8 (0000-01-kquant-integer-dpas.patch:1862-1889): scale bm/127, codes
    round-to-nearest-even of v*127/bm, zero block below 1e-30, integer sums per 32."""
    x = O.fill_normal(4 * 512, 3, 1.0).reshape(4, 512)
    x[1, :256] = 0.0
    x[2, :256] = 1e-35
    q, d, s = O.quantize_act_q8_256(x)
    for c in range(4):
        for b in range(2):
            blk = x[c, 256 * b:256 * b + 256]
            bm = np.abs(blk).max()
            assert d[c, b] == np.float32(bm) / np.float32(127)
            iq = np.float32(127) / bm if bm > 1e-30 else np.float32(0)
            assert np.array_equal(q[c, 256 * b:256 * b + 256], np.rint(blk * iq).astype(np.int8))
    assert np.array_equal(s, q.reshape(4, 16, 32).astype(np.int32).sum(-1).astype(np.int16))
    assert np.abs(q).max() == 127 and not q[1, :256].any() and not q[2, :256].any()


def test_rounding_half_away_at_scale_one():
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, :8] = [127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 0.49]
    q, d = O.quantize_act_q8_0(x)
    assert d[0, 0] == np.float16(1.0).view(np.uint16)
    assert list(q[0, :8]) == [127, 1, -1, 2, -2, 3, -3, 0]


def _fp64_ref(t, w, k, x, quantized):
    wd = O.dequantize(t, w, k).astype(np.float64)
    if quantized:
        if O.act_form(t) == O.ACT_Q8_0:
            q, d = O.quantize_act_q8_0(x)
            xa = q.astype(np.float64) * np.repeat(d.view(np.float16).astype(np.float64), 32, axis=1)
        else:
            q, d, _ = O.quantize_act_q8_256(x)
            xa = q.astype(np.float64) * np.repeat(d.astype(np.float64), 256, axis=1)
    else:
        xa = x.astype(np.float64)
    return xa @ wd.T


def rel_err(got, ref):
    """max relative error per column against max(|ref|, 1e-2 * max|ref| of the column)"""
    ref = np.asarray(ref, dtype=np.float64)
    floor = 1e-2 * np.abs(ref).max(axis=-1, keepdims=True)
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), floor)).max())


@pytest.mark.parametrize("t", O.QUANT_TYPES)
def test_mul_mat_against_numpy_fp64(t):
    rng = np.random.default_rng(t)
    m, k, n = 24, 512, 5
    w = O.quantize(t, O.fill_normal(m * k, 11 + t, 0.02).reshape(m, k))
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    ref = _fp64_ref(t, w, k, x, True)
    assert np.allclose(O.mul_mat_f64(t, w, k, x, True), ref, rtol=1e-12, atol=1e-12)
    assert np.allclose(O.mul_mat_f64(t, w, k, x, False), _fp64_ref(t, w, k, x, False), rtol=1e-12, atol=1e-12)
    got = O.mul_mat(t, w, k, x)
    assert rel_err(got, ref) < 1e-4
    # against raw f32 activations the int8 rounding shows, but stays small (NMSE bound of the reference's op suite)
    raw = _fp64_ref(t, w, k, x, False)
    nmse = ((got - raw) ** 2).sum() / (raw ** 2).sum()
    assert nmse < 5e-4


@pytest.mark.parametrize("t", O.QUANT_TYPES)
def test_mul_mat_random_field_blocks(t):
    rng = np.random.default_rng(100 + t)
    m, k, n = 16, 768 if O.block_size(t) == 256 else 96, 3
    w = O.random_blocks(t, m, k, rng)
    x = rng.normal(0, 1, size=(n, k)).astype(np.float32)
    assert rel_err(O.mul_mat(t, w, k, x), _fp64_ref(t, w, k, x, True)) < 1e-4


def test_mul_mat_threads_agree():
    t, m, k, n = O.Q4_K, 40, 512, 4
    w = O.quantize(t, O.fill_normal(m * k, 5, 0.02).reshape(m, k))
    x = O.fill_normal(n * k, 6, 1.0).reshape(n, k)
    assert np.array_equal(O.mul_mat(t, w, k, x, nthreads=1), O.mul_mat(t, w, k, x, nthreads=0))


def test_mul_mat_id_column_rule_and_views():
    t, m, k, n_expert, n_used, n_tok = O.Q4_K, 8, 256, 6, 3, 5
    rng = np.random.default_rng(9)
    w = np.stack([O.random_blocks(t, m, k, rng) for _ in range(n_expert)])
    ids_full = rng.integers(0, n_expert, size=(n_tok, n_used + 2), dtype=np.int32)
    ids_full[2, 2:5] = 4                                   # duplicate ids within a token
    ids = ids_full[:, 2:]                                  # ids through an offset view
    for ne11 in (1, n_used):
        x = rng.normal(0, 1, size=(n_tok, ne11, k)).astype(np.float32)
        got = O.mul_mat_id(t, w, m, k, x, ids)
        for tok in range(n_tok):
            for i in range(n_used):
                want = O.mul_mat(t, w[ids[tok, i]], k, x[tok, i % ne11][None])[0]
                assert np.array_equal(got[tok, i], want)
    with pytest.raises(ValueError):
        bad = ids.copy()
        bad[0, 0] = n_expert
        O.mul_mat_id(t, w, m, k, x, bad)


def test_moe_route_tiles():
    rng = np.random.default_rng(4)
    n_expert, n_used, n_tok, tile = 17, 4, 50, 8
    ids = rng.integers(0, n_expert, size=(n_tok, n_used), dtype=np.int32)
    pairs, tiles = O.moe_route(ids, n_expert, tile)
    flat = ids.reshape(-1)
    assert sorted(pairs.tolist()) == list(range(n_tok * n_used))
    assert np.all(np.diff(flat[pairs]) >= 0)               # sorted by expert
    pos = 0
    for e, first, count, _ in tiles:
        assert first == pos and 0 < count <= tile
        assert np.all(flat[pairs[first:first + count]] == e)
        pos += count
    assert pos == n_tok * n_used
    assert len(tiles) <= -(-n_tok * n_used // tile) + min(n_expert, n_tok * n_used)


def test_route_ids_properties():
    ids = O.route_ids(10, 64, 512, 123)
    assert ids.shape == (64, 10) and ids.min() >= 0 and ids.max() < 512
    assert all(len(set(r)) == 10 for r in ids.tolist())
    counts = np.bincount(ids.reshape(-1), minlength=512)
    assert counts.max() > 8 * np.median(counts[counts > 0])   # skewed popularity
    assert (counts > 0).sum() > 100                           # ... with a long tail


def test_fill_normal_is_seeded():
    a, b, c = O.fill_normal(10001, 42, 0.02), O.fill_normal(10001, 42, 0.02), O.fill_normal(10001, 43, 0.02)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert abs(a.std() - 0.02) < 1e-3 and abs(a.mean()) < 1e-3


# ---- against the reference's own text (kq_i8_ops.inc), when it was built ----

needs_ref = pytest.mark.skipif(O.ref() is None, reason="oracle/_ref not built (reference tree absent)")


@needs_ref
def test_ref_iq4nl_decode_matches_oracle_and_golden(golden):
    R = O.ref()
    blocks = golden["iq4_xs_blocks"].reshape(-1, 136)
    deq = golden["iq4_xs_deq"].reshape(-1, 256)
    for bi in range(blocks.shape[0]):
        b = blocks[bi]
        d = b[:2].view(np.float16).astype(np.float32)[0]
        sh = int(b[2:4].view(np.uint16)[0])
        for p in range(8):
            out = np.zeros(32, dtype=np.int8)
            qs = np.ascontiguousarray(b[8 + 16 * p: 8 + 16 * p + 16])
            R.ref_kq_i8_decode_iq4nl(qs.ctypes.data, O.KVALUES_IQ4NL.ctypes.data, out.ctypes.data)
            ls = ((int(b[4 + p // 2]) >> (4 * (p & 1))) & 0xF) | (((sh >> (2 * p)) & 3) << 4)
            want = (d * np.float32(ls - 32)) * out.astype(np.float32)
            assert np.array_equal(want, deq[bi, 32 * p:32 * p + 32])


@needs_ref
def test_ref_quant32_same_grid():
    """kq_i8_quant32 uses 127/amax as the inverse where ggml uses 1/(amax/127): the codes
    agree except on rare last-place ties, never by more than one step; scales agree after
    the fp16 rounding ggml's block stores."""
    R = O.ref()
    x = O.fill_normal(32 * 4000, 77, 1.0).reshape(4000, 32)
    q, d = O.quantize_act_q8_0(x)
    rq = np.zeros((4000, 32), dtype=np.int8)
    rd = np.zeros(4000, dtype=np.float32)
    for i in range(4000):
        R.ref_kq_i8_quant32(x[i].ctypes.data, rq[i].ctypes.data, rd[i:].ctypes.data)
    diff = np.abs(q.astype(np.int32) - rq.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    assert np.array_equal(rd.astype(np.float16).view(np.uint16), d[:, 0])
    # the reference's own pins: .5 away from zero at scale 1, amax/127 scale
    t = np.zeros(32, dtype=np.float32)
    t[:5] = [127.0, 0.5, -0.5, 2.5, -2.5]
    R.ref_kq_i8_quant32(t.ctypes.data, rq[0].ctypes.data, rd.ctypes.data)
    assert list(rq[0, :5]) == [127, 1, -1, 3, -3] and rd[0] == 1.0
    qq, _ = O.quantize_act_q8_0(t[None])
    assert np.array_equal(qq[0], rq[0])


@needs_ref
def test_ref_column_rule():
    R = O.ref()
    for n_used, ne11 in ((10, 1), (10, 10), (4, 2), (1, 1)):
        for p in range(3 * n_used):
            t, i = divmod(p, n_used)
            assert R.ref_kq_i8_col(p, n_used, ne11) == (i % ne11) + t * ne11
