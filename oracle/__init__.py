"""ctypes/numpy wrapper around the CPU oracle (liborc.so) and, when built, the
reference's own kq_i8_ops.inc (_ref/libkqref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs, as the checker. The product package never imports it.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))

F32, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS, I32 = 0, 2, 8, 12, 13, 14, 20, 23, 26
QUANT_TYPES = (Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS, IQ4_NL)
TYPE_NAMES = {Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_K", Q5_K: "q5_K", Q6_K: "q6_K", IQ4_XS: "iq4_xs", IQ4_NL: "iq4_nl"}
ACT_Q8_0, ACT_Q8_256 = 0, 1
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.int8)

_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        so = os.path.join(HERE, "liborc.so")
        if not os.path.exists(so):
            so = _build.build_oracle()
        L = C.CDLL(so)
        i64, vp, ci = C.c_int64, C.c_void_p, C.c_int
        L.orc_block_size.restype = ci
        L.orc_block_bytes.restype = C.c_size_t
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [ci, i64]
        L.orc_fp16_to_fp32.restype = C.c_float
        L.orc_fp16_to_fp32.argtypes = [C.c_uint16]
        L.orc_fp32_to_fp16.restype = C.c_uint16
        L.orc_fp32_to_fp16.argtypes = [C.c_float]
        L.orc_dequantize_row.argtypes = [ci, vp, vp, i64]
        L.orc_quantize_rows.argtypes = [ci, vp, vp, i64, i64, ci]
        L.orc_quantize_act_q8_0.argtypes = [vp, vp, vp, i64]
        L.orc_quantize_act_q8_256.argtypes = [vp, vp, vp, vp, i64]
        L.orc_mul_mat.argtypes = [ci, vp, i64, i64, vp, i64, i64, vp, i64, ci]
        L.orc_mul_mat_f64.argtypes = [ci, vp, i64, i64, vp, i64, i64, vp, i64, ci, ci]
        L.orc_mul_mat_id.argtypes = [ci, vp, i64, i64, ci, vp, ci, ci, vp, i64, ci, vp, ci]
        L.orc_mul_mat_id_f64.argtypes = [ci, vp, i64, i64, ci, vp, ci, ci, vp, i64, ci, vp, ci, ci]
        L.orc_moe_route.argtypes = [vp, i64, ci, ci, ci, ci, vp, vp]
        L.orc_fill_normal.argtypes = [vp, i64, C.c_uint64, C.c_float, ci]
        L.orc_route_ids.argtypes = [vp, ci, ci, ci, C.c_uint64, C.c_float]
        _lib = L
    return _lib


def ref():
    """The reference's kq_i8_ops.inc behind a C shim, or None when it was never built."""
    global _ref
    if _ref is None:
        so = os.path.join(HERE, "_ref", "libkqref.so")
        if not os.path.exists(so):
            return None
        R = C.CDLL(so)
        R.ref_kq_i8_quant32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        R.ref_kq_i8_decode_iq4nl.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        R.ref_kq_i8_col.argtypes = [C.c_int, C.c_int, C.c_int]
        R.ref_kq_i8_col.restype = C.c_int
        R.ref_kq_i8_mean_pairs.argtypes = [C.c_long, C.c_int]
        R.ref_kq_i8_mean_pairs.restype = C.c_long
        _ref = R
    return _ref


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def block_size(t):
    return lib().orc_block_size(t)


def block_bytes(t):
    return lib().orc_block_bytes(t)


def row_bytes(t, k):
    return lib().orc_row_bytes(t, k)


def act_form(t):
    return ACT_Q8_0 if t in (Q4_0, Q8_0, IQ4_NL) else ACT_Q8_256


def num_threads():
    return lib().orc_num_threads()


def fill_normal(n, seed, sigma=1.0):
    out = np.empty(int(n), dtype=np.float32)
    lib().orc_fill_normal(_p(out), out.size, seed, sigma, 0)
    return out


def quantize(t, w):
    """w: f32 [rows, k] -> uint8 [rows, row_bytes]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    out = np.empty((rows, row_bytes(t, k)), dtype=np.uint8)
    rc = lib().orc_quantize_rows(t, _p(w), _p(out), rows, k, 0)
    if rc:
        raise ValueError("orc_quantize_rows: %d" % rc)
    return out


def dequantize(t, blocks, k):
    """blocks: uint8 [rows, row_bytes] -> f32 [rows, k]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rows = blocks.shape[0]
    out = np.empty((rows, k), dtype=np.float32)
    for r in range(rows):
        rc = lib().orc_dequantize_row(t, _p(blocks[r]), _p(out[r]), k)
        if rc:
            raise ValueError("orc_dequantize_row: %d" % rc)
    return out


def quantize_act_q8_0(x):
    """x: f32 [n, k] -> (int8 [n,k], fp16-bits uint16 [n,k/32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = x.shape
    q = np.empty((n, k), dtype=np.int8)
    d = np.empty((n, k // 32), dtype=np.uint16)
    for c in range(n):
        lib().orc_quantize_act_q8_0(_p(x[c]), _p(q[c]), _p(d[c]), k)
    return q, d


def quantize_act_q8_256(x):
    """x: f32 [n, k] -> (int8 [n,k], f32 [n,k/256], int16 sums [n,k/32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = x.shape
    q = np.empty((n, k), dtype=np.int8)
    d = np.empty((n, k // 256), dtype=np.float32)
    s = np.empty((n, k // 32), dtype=np.int16)
    for c in range(n):
        lib().orc_quantize_act_q8_256(_p(x[c]), _p(q[c]), _p(d[c]), _p(s[c]), k)
    return q, d, s


def mul_mat(t, w, k, x, nthreads=0):
    """w: uint8 [m, row_bytes]; x: f32 [n, k] (one row per column of src1) -> f32 [n, m]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, n = w.shape[0], x.shape[0]
    out = np.empty((n, m), dtype=np.float32)
    rc = lib().orc_mul_mat(t, _p(w), m, k, _p(x), n, k, _p(out), m, nthreads)
    if rc:
        raise ValueError("orc_mul_mat: %d" % rc)
    return out


def mul_mat_f64(t, w, k, x, quantized_act=True, nthreads=0):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, n = w.shape[0], x.shape[0]
    out = np.empty((n, m), dtype=np.float64)
    rc = lib().orc_mul_mat_f64(t, _p(w), m, k, _p(x), n, k, _p(out), m, int(quantized_act), nthreads)
    if rc:
        raise ValueError("orc_mul_mat_f64: %d" % rc)
    return out


def mul_mat_id(t, w, m, k, x, ids, f64=False, quantized_act=True, nthreads=0):
    """w: uint8 [n_expert, m, row_bytes]; x: f32 [n_tok, ne11, k]; ids: int32 [n_tok, n_used]
    (may be a strided view along axis 0) -> [n_tok, n_used, m]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n_expert = w.shape[0]
    n_tok, ne11, _ = x.shape
    n_used = ids.shape[1]
    assert ids.dtype == np.int32 and ids.strides[1] == 4 and ids.strides[0] % 4 == 0
    stride = ids.strides[0] // 4
    out = np.empty((n_tok, n_used, m), dtype=np.float64 if f64 else np.float32)
    if f64:
        rc = lib().orc_mul_mat_id_f64(t, _p(w), m, k, n_expert, _p(x), ne11, n_tok, C.c_void_p(ids.ctypes.data),
                                      stride, n_used, _p(out), int(quantized_act), nthreads)
    else:
        rc = lib().orc_mul_mat_id(t, _p(w), m, k, n_expert, _p(x), ne11, n_tok, C.c_void_p(ids.ctypes.data),
                                  stride, n_used, _p(out), nthreads)
    if rc:
        raise ValueError("orc_mul_mat_id: %d" % rc)
    return out


def moe_route(ids, n_expert, tile):
    """ids int32 [n_tok, n_used] -> (pairs int32 [n_pairs], tiles int32 [n_tiles, 4])."""
    n_tok, n_used = ids.shape
    assert ids.dtype == np.int32 and ids.strides[1] == 4
    n_pairs = n_tok * n_used
    pairs = np.empty(n_pairs, dtype=np.int32)
    max_tiles = (n_pairs + tile - 1) // tile + min(n_expert, n_pairs)
    tiles = np.zeros((max_tiles, 4), dtype=np.int32)
    nt = lib().orc_moe_route(C.c_void_p(ids.ctypes.data), ids.strides[0] // 4, n_used, n_tok, n_expert, tile,
                             _p(pairs), _p(tiles))
    if nt < 0:
        raise ValueError("orc_moe_route: %d" % nt)
    return pairs, tiles[:nt]


def route_ids(n_used, n_tok, n_expert, seed, zipf_s=1.1):
    ids = np.empty((n_tok, n_used), dtype=np.int32)
    lib().orc_route_ids(_p(ids), n_used, n_tok, n_expert, seed, zipf_s)
    return ids


def random_blocks(t, rows, k, rng):
    """Random-field blocks with sane fp16 scales (the reference's own test method,
    0000-09-moe-routing-gemm-tiles.patch:1143-1150): every code byte random, every
    fp16 scale a finite value of modest size."""
    bs, bb = block_size(t), block_bytes(t)
    nb = k // bs
    raw = rng.integers(0, 256, size=(rows, nb, bb), dtype=np.uint8)

    def put_half(off, lo, hi, signed=True):
        v = rng.uniform(lo, hi, size=(rows, nb)).astype(np.float32)
        if signed:
            v *= rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=(rows, nb))
        h = v.astype(np.float16).view(np.uint16)
        raw[:, :, off] = (h & 0xFF).astype(np.uint8)
        raw[:, :, off + 1] = (h >> 8).astype(np.uint8)

    if t in (Q4_0, Q8_0, IQ4_XS, IQ4_NL):
        put_half(0, 1e-3, 2e-2)
    elif t in (Q4_K, Q5_K):
        put_half(0, 1e-4, 2e-3, signed=False)
        put_half(2, 1e-4, 2e-3, signed=False)
    elif t == Q6_K:
        put_half(208, 1e-5, 5e-4)
    return raw.reshape(rows, nb * bb)


def moe_router(logits, n_used, cmin, cmax):
    """The MoE router as the reference's fused kernel computes it (kernel_topk_moe_softmax_norm_n*,
    0000-09-moe-routing-gemm-tiles.patch:928-987): per token p = exp(x - max x), s = sum p, the n_used
    largest p in descending order (ties: the lower expert id), w_j = p_j / s, then w_j / clamp(sum_j w_j,
    cmin, cmax). logits: f32 [n_tok, n_expert] -> ids int32 [n_tok, n_used], weights f32 [n_tok, n_used]."""
    x = np.asarray(logits, dtype=np.float32)
    p = np.exp(x - x.max(axis=1, keepdims=True)).astype(np.float32)
    s = p.sum(axis=1, dtype=np.float64).astype(np.float32)
    order = np.argsort(-p, axis=1, kind="stable")[:, :n_used]          # stable: equal values keep the lower id first
    w = (np.take_along_axis(p, order, axis=1) / s[:, None]).astype(np.float32)
    denom = np.clip(w.sum(axis=1, dtype=np.float32), np.float32(cmin), np.float32(cmax))
    return order.astype(np.int32), (w / denom[:, None]).astype(np.float32)


def moe_ffn(t, gate_w, up_w, down_w, d_model, d_ff, x, logits, n_used, cmin, cmax):
    """The feed-forward block around MUL_MAT_ID in fp64 on the library's quantized operands: router, gate and up
    over x [n_tok, d_model], h = silu(gate) * up (rounded to f32, as the block hands it to the down projection),
    down, and the weighted sum over the used experts -> (y [n_tok, d_model] f64, ids, weights)."""
    ids, w = moe_router(logits, n_used, cmin, cmax)
    x3 = np.ascontiguousarray(x, dtype=np.float32)[:, None, :]
    g = mul_mat_id(t, gate_w, d_ff, d_model, x3, ids, f64=True)
    u = mul_mat_id(t, up_w, d_ff, d_model, x3, ids, f64=True)
    h = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    d = mul_mat_id(t, down_w, d_model, d_ff, h, ids, f64=True)
    return (d * w[:, :, None].astype(np.float64)).sum(axis=1), ids, w
